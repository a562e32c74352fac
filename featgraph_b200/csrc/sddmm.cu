// COO SDDMM for sm_100a, single- and multi-head:
//   out[e, h] = sum_{d<D} src[col[e], h*D+d] * dst[row[e], h*D+d]
//
// The sum over d runs in ascending order in one fp32 accumulator with the
// product and the sum rounded separately -- the order of the reference's
// unscheduled reduction (python/featgraph/op/vanilla_sddmm.py:43-47, 66-74) --
// so results are bit-equal to a sequential loop.
//
// sddmm_tile_kernel: each warp owns 32 consecutive edges per tile.  The
// gathered feature rows are staged, 32 floats at a time, into shared memory with
// 16-byte cp.async copies in which 8 lanes read one 128-byte row segment
// (coalesced gathers); latency is hidden by the 36 warps an SM holds, not by a
// ring per warp.  Each lane then walks ITS edge's two
// segments with float4 shared-memory loads (row pitch 36 floats, conflict
// free) and adds the products in order.  Runs of consecutive edges with the
// same row (the normal case for a row-sorted COO list) stage dst[row] once per
// run and read it back as a broadcast.
//
// sddmm_rowreg_kernel: one head over a list with long runs of equal rows -- the dst
// operand stays in registers across four tiles (chosen by a launch hint).
// sddmm_tma_kernel: the tile kernel's arithmetic with the gathers done by TMA tile::gather4
// copies (a launch option; slower on B200 for 128-byte segments).
//
// sddmm_generic_kernel: any shape / alignment, one thread per (edge, head).
#include <cuda.h>  // CUtensorMap and the enums of cuTensorMapEncodeTiled (types only; no libcuda link)

#include <algorithm>

#include "common.cuh"

namespace fg {

constexpr int kSdChunk = 32;             // floats per row per stage
constexpr int kSdPitch = kSdChunk + 4;   // smem row pitch (floats): conflict-free LDS.128
constexpr int kSdWarps = 6;              // warps per CTA
// Stages per warp.  One: a warp copies a stage, waits, consumes it.  Measured on B200
// (114.6 M edges, feat_len 64): 1 stage x 36 warps/SM 2.76 ms, 2 x 18 3.21 ms, 3 x 12
// 3.94 ms -- a warp keeps only a few cp.async copies outstanding however deep its
// ring, so shared memory is better spent on more warps than on deeper rings.
constexpr int kSdStages = 1;
constexpr int kSdDstSlots = 8;           // distinct dst rows a stage can hold
// one stage: src segments of 32 edges, dst segments of up to 8 distinct rows, then
// 32 per-lane words (slot id, or the row itself) and the 8 row ids of the slots
constexpr int kSdStageFloats = 32 * kSdPitch + kSdDstSlots * kSdPitch + 32 + kSdDstSlots;
constexpr int kSdWarpFloats = kSdStages * kSdStageFloats;
constexpr int kSdSmemBytes = kSdWarps * kSdWarpFloats * 4;
static_assert(kSdStageFloats % 4 == 0, "stages stay 16-byte aligned");

constexpr int kSdTilesPerWarpConst = 16;             // tiles a warp walks (kSdTilesPerWarp)
constexpr int kSdLanesPerSeg = kSdChunk / 4;          // 16-byte copies per row segment
constexpr int kSdRowsPerCopy = 32 / kSdLanesPerSeg;   // segments one warp-wide copy covers

// HEAD_DIM: the head size D when a head ends inside a chunk (D = 4, 8, ... up to
// the chunk size), or 0 when D is a larger multiple of the chunk (heads end only at
// chunk boundaries).
// MSG / RED: the message and reduce operators (FG_MSG_MUL with FG_REDUCE_SUM is the dot
// product of the reference; lhs = the src element, rhs = the dst element).
template <int HEAD_DIM, int MSG, int RED>
__global__ void __launch_bounds__(kSdWarps * 32)
sddmm_tile_kernel(const int* __restrict__ row, const int* __restrict__ col,
                  const float* __restrict__ src, const float* __restrict__ dst,
                  const __grid_constant__ OutPtrs out, long long nnz, int F, int H,
                  int tiles_per_warp, int vec_heads) {
  constexpr unsigned kFull = 0xffffffffu;
  extern __shared__ __align__(16) float smem[];
  launch_dependents();  // a kernel launched programmatically behind this one may be dispatched
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float* wbuf = smem + warp * kSdWarpFloats;

  const long long n_tiles = (nnz + 31) / 32;
  const long long tile0 = ((long long)blockIdx.x * kSdWarps + warp) * tiles_per_warp;
  // (warp 0 of every CTA has tiles, so the wait at the end of the last CTA is always reached)
  if (tile0 >= n_tiles) return;
  const int my_tiles = (int)min((long long)tiles_per_warp, n_tiles - tile0);
  const int n_chunks = F / kSdChunk;
  const int total = my_tiles * n_chunks;
  const int chunks_per_head = HEAD_DIM == 0 ? (F / H) / kSdChunk : 1;

  // State of the tile being issued: one edge per lane, and the tile's runs of
  // equal row index.  Edge lists sorted by row repeat dst[row] for hundreds of
  // consecutive edges; each distinct run is staged once ("slot") and the lanes of
  // the run read it back as a shared-memory broadcast.  A tile with more than
  // kSdDstSlots runs (an unsorted list, or very short rows) stages no dst rows:
  // its lanes read their dst segments straight from global memory instead.
  int r_iss = 0, c_iss = 0, word_iss = 0, n_slots = 1;
  bool head_iss = false;
  // Indices of the tile after the one being issued, fetched a whole tile ahead
  // so that their DRAM latency never stalls the copy pipeline.
  int r_ahead = 0, c_ahead = 0;
  auto fetch_indices = [&](int t) {
    const long long e = (tile0 + t) * 32 + lane;
    r_ahead = 0;
    c_ahead = 0;
    if (t < my_tiles && e < nnz) {
      r_ahead = ld_stream(row + e);
      c_ahead = ld_stream(col + e);
    }
  };
  auto begin_tile = [&](int t) {
    r_iss = r_ahead;
    c_iss = c_ahead;
    fetch_indices(t + 1);
    const int r_left = __shfl_up_sync(kFull, r_iss, 1);
    head_iss = lane == 0 || r_iss != r_left;
    const unsigned run_heads = __ballot_sync(kFull, head_iss);
    n_slots = __popc(run_heads);
    const int slot = __popc(run_heads & (0xffffffffu >> (31 - lane))) - 1;
    // per-lane word: slot id (>= 0), or -1 - row when the tile reads dst directly
    word_iss = n_slots <= kSdDstSlots ? slot : -1 - r_iss;
  };
  // Stage (tile t_iss, chunk ch_iss) into buffer `buf`.
  int t_iss = 0, ch_iss = 0;
  auto issue = [&](int buf) {
    if (ch_iss == 0) begin_tile(t_iss);
    float* sbuf = wbuf + buf * kSdStageFloats;
    float* dbuf = sbuf + 32 * kSdPitch;
    int* words = reinterpret_cast<int*>(dbuf + kSdDstSlots * kSdPitch);
    int* slot_rows = words + 32;
    const bool staged = n_slots <= kSdDstSlots;
    words[lane] = word_iss;
    if (staged && head_iss) slot_rows[word_iss] = r_iss;
    __syncwarp();
    const int part = (lane % kSdLanesPerSeg) * 4;
    const size_t foff = (size_t)ch_iss * kSdChunk + part;
    const float* sp = src + foff;
#pragma unroll
    for (int k = 0; k < 32 / kSdRowsPerCopy; ++k) {
      const int e = lane / kSdLanesPerSeg + kSdRowsPerCopy * k;
      const int c = __shfl_sync(kFull, c_iss, e);
      // .cg (no L1 allocation) although ncu shows that the bypass path brings 24 sectors per
      // warp-wide copy across the crossbar where the four 128-byte segments hold 16 (.ca
      // brings exactly 16): with .ca the kernel is SLOWER (3.55 against 2.81 ms at feat 64) --
      // the L1's allocation work costs more than the extra sectors.  Loading the segments
      // into registers and storing them with STS.128 (4 shared-memory wavefronts per warp-wide
      // store where a cp.async deposit takes 9.5) is slower still: 4.3 to 6.1 ms with 30 to 24
      // warps per SM -- the copy has to be asynchronous
      cp_async16_cg(sbuf + e * kSdPitch + part, sp + (size_t)c * F);
    }
    if (staged) {
#pragma unroll
      for (int k = 0; k < (kSdDstSlots + kSdRowsPerCopy - 1) / kSdRowsPerCopy; ++k) {
        const int slot = lane / kSdLanesPerSeg + kSdRowsPerCopy * k;
        if (slot < n_slots)
          cp_async16_ca(dbuf + slot * kSdPitch + part, dst + (size_t)slot_rows[slot] * F + foff);
      }
    }
    if (++ch_iss == n_chunks) {
      ch_iss = 0;
      ++t_iss;
    }
  };

  fetch_indices(0);
#pragma unroll
  for (int p = 0; p < kSdStages - 1; ++p) {
    if (p < total) issue(p);
    cp_async_commit();
  }
  float acc = red_identity<RED>();
  int head = 0, chunk = 0, buf = 0, buf_issue = kSdStages - 1;
  long long e = tile0 * 32 + lane;
  // A finished head leaves at once (one 4-byte store per lane: a warp's 32 edges lie H
  // floats apart), or, when H is a multiple of four (vec_heads), waits for three more so
  // that the lane stores 16 contiguous bytes -- a quarter of the store instructions and
  // whole sectors instead of 4-byte pieces of them.
  float4 pend = make_float4(0.f, 0.f, 0.f, 0.f);
  auto finish_head = [&]() {
    if (vec_heads) {
      switch (head & 3) {
        case 0: pend.x = acc; break;
        case 1: pend.y = acc; break;
        case 2: pend.z = acc; break;
        default:
          pend.w = acc;
          if (e < nnz) out_store(out, (size_t)e * H + head - 3, pend);
      }
    } else if (e < nnz) {
      out_store(out, (size_t)e * H + head, acc);
    }
    ++head;
    acc = red_identity<RED>();
  };
  for (int it = 0; it < total; ++it) {
    if (it + kSdStages - 1 < total) issue(buf_issue);
    cp_async_commit();
    cp_async_wait<kSdStages - 1>();
    __syncwarp();

    const float* stage = wbuf + buf * kSdStageFloats;
    const int word = reinterpret_cast<const int*>(stage + (32 + kSdDstSlots) * kSdPitch)[lane];
    const float4* s4 = reinterpret_cast<const float4*>(stage + lane * kSdPitch);
    // word >= 0: this lane's dst segment is slot `word` of the stage; otherwise it
    // is row -1 - word of dst in global memory (uniform across the warp)
    const float4* d4 =
        word >= 0 ? reinterpret_cast<const float4*>(stage + (32 + word) * kSdPitch)
                  : reinterpret_cast<const float4*>(dst + (size_t)(-1 - word) * F +
                                                    (size_t)chunk * kSdChunk);
#pragma unroll
    for (int q = 0; q < kSdChunk / 4; ++q) {
      const float4 a = s4[q];
      const float4 b = d4[q];
      acc = combine<MSG, RED>(acc, a.x, b.x);
      acc = combine<MSG, RED>(acc, a.y, b.y);
      acc = combine<MSG, RED>(acc, a.z, b.z);
      acc = combine<MSG, RED>(acc, a.w, b.w);
      if (HEAD_DIM > 0 && ((q + 1) * 4) % (HEAD_DIM > 0 ? HEAD_DIM : 4) == 0) finish_head();
    }
    ++chunk;
    if (HEAD_DIM == 0 && chunk % chunks_per_head == 0) finish_head();
    if (chunk == n_chunks) {  // next stage belongs to the next tile
      chunk = 0;
      head = 0;
      acc = red_identity<RED>();
      e += 32;
    }
    buf = buf == kSdStages - 1 ? 0 : buf + 1;
    buf_issue = buf_issue == kSdStages - 1 ? 0 : buf_issue + 1;
    __syncwarp();  // every lane is done with this buffer before it is refilled
  }
  cp_async_wait<0>();
  // If this grid was dispatched behind another one without waiting for it (programmatic
  // launch), its last CTA stays until that one has completed: "this grid is complete" then
  // covers both for whatever follows in the stream.
  if (blockIdx.x == gridDim.x - 1 && warp == 0) wait_for_prior_grids();
}

// ---- single-head tiles with the dst operand in registers -----------------------------
//
// sddmm_rowreg_kernel (one head, feat_len a multiple of 32).  In sddmm_tile_kernel a lane
// fetches BOTH operands of its edge through the LSU: per 32-edge x 32-float stage the
// lanes' loads of the dst segment cost as many shared-memory wavefronts as the loads of
// their own src row (a 16-byte load returns 512 bytes to the warp even when every lane
// reads the same address), 67 of the stage's 96, and that pipe is what bounds the kernel
// (84 % busy).  A row-sorted edge list repeats dst[row] for hundreds of consecutive edges,
// so here the dst segment lives in REGISTERS: a warp takes its tiles four at a time, walks
// the feature axis in the OUTER loop and the four tiles in the inner one, and loads the 32
// floats of dst[row] for the current chunk once per group of tiles whose edges all share
// that row (eight 16-byte loads with one address).  The four partial sums wait in
// registers for the next chunk; the order of the additions per edge is unchanged (k
// ascending), so the results are sddmm_tile_kernel's bit for bit.  A tile that crosses a
// row boundary reads its lanes' dst segments from global memory (L1) instead.
// Two stages per warp: the copies of the next (tile, chunk) are in flight while the
// current one is summed.
// Measured on B200 (114.6 M edges, feat_len 64, ms; sddmm_tile_kernel: 2.82): 4 warps x 4
// CTAs per SM (128 registers), groups of 4 tiles, 2 stages: 2.64; 5 CTAs (96 registers, a few
// spills): 2.65; 6 CTAs (80 registers): 3.37; 3 stages: 2.74; 6 warps x 3 CTAs: 2.70; groups
// of 8 tiles: 3.10; L1-allocating copies (.ca): 2.74 (better only from feat_len 256 up).
constexpr int kRrWarps = 4;
constexpr int kRrMinCtas = 4;
constexpr int kRrTiles = 4;              // tiles per group (partial sums held in registers)
constexpr int kRrStages = 2;
constexpr int kRrAhead = kRrStages - 1;  // stages in flight beyond the one being summed
static_assert(kRrAhead >= 1 && kRrAhead <= kRrTiles, "prefetch distance");
constexpr int kRrStageFloats = 32 * kSdPitch;
constexpr int kRrSmemBytes = kRrWarps * kRrStages * kRrStageFloats * 4;
static_assert(kSdTilesPerWarpConst % kRrTiles == 0, "a warp's tiles split into whole groups");

template <int MSG, int RED>
__global__ void __launch_bounds__(kRrWarps * 32, kRrMinCtas)
sddmm_rowreg_kernel(const int* __restrict__ row, const int* __restrict__ col,
                    const float* __restrict__ src, const float* __restrict__ dst,
                    const __grid_constant__ OutPtrs out, long long nnz, int F,
                    int tiles_per_warp) {
  constexpr unsigned kFull = 0xffffffffu;
  extern __shared__ __align__(16) float rr_smem[];
  launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  float* wbuf = rr_smem + warp * kRrStages * kRrStageFloats;

  const long long n_tiles = (nnz + 31) / 32;
  const long long tile0 = ((long long)blockIdx.x * kRrWarps + warp) * tiles_per_warp;
  if (tile0 >= n_tiles) return;  // (warp 0 of every CTA has tiles)
  const int n_chunks = F / kSdChunk;
  const int part = (lane % kSdLanesPerSeg) * 4;
  const int e_lo = lane / kSdLanesPerSeg;

  // tiles past the end of the list are walked as empty ones (indices 0, nothing stored),
  // so that every group is whole
  for (int g0 = 0; g0 < tiles_per_warp && tile0 + g0 < n_tiles; g0 += kRrTiles) {
    int cidx[kRrTiles], ridx[kRrTiles], row0[kRrTiles];
    bool one_run[kRrTiles];
    float acc[kRrTiles];
#pragma unroll
    for (int j = 0; j < kRrTiles; ++j) {
      const long long e = (tile0 + g0 + j) * 32 + lane;
      cidx[j] = 0;
      ridx[j] = 0;
      if (e < nnz) {
        ridx[j] = ld_stream(row + e);
        cidx[j] = ld_stream(col + e);
      }
      acc[j] = red_identity<RED>();
    }
    // ask L2 for the next group's indices, so that its loads find them there (the group's
    // first copies wait for them: 1.52 -> 1.45 ms at feat_len 32, about 1 % from 64 up;
    // holding them in registers a group ahead instead was no faster)
    if (g0 + kRrTiles < tiles_per_warp) {
#pragma unroll
      for (int j = 0; j < kRrTiles; ++j) {
        const long long e = (tile0 + g0 + kRrTiles + j) * 32 + lane;
        if (e < nnz) {
          asm volatile("prefetch.global.L2 [%0];" ::"l"(row + e));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(col + e));
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kRrTiles; ++j) {
      row0[j] = __shfl_sync(kFull, ridx[j], 0);
      one_run[j] = __all_sync(kFull, ridx[j] == row0[j]);
    }
    // copies of (tile j, chunk ch) into stage buffer `buf`
    auto issue = [&](int cj, int ch, int buf) {
      float* sbuf = wbuf + buf * kRrStageFloats;
      const float* sp = src + (size_t)ch * kSdChunk + part;
#pragma unroll
      for (int k = 0; k < 32 / kSdRowsPerCopy; ++k) {
        const int e = e_lo + kSdRowsPerCopy * k;
        const int c = __shfl_sync(kFull, cj, e);
        cp_async16_cg(sbuf + e * kSdPitch + part, sp + (size_t)c * F);
      }
      cp_async_commit();
    };
#pragma unroll
    for (int j = 0; j < kRrAhead; ++j) issue(cidx[j], 0, j);
    int buf = 0;
    for (int ch = 0; ch < n_chunks; ++ch) {
      float4 b[kSdChunk / 4];
      int have_row = -1;
#pragma unroll
      for (int j = 0; j < kRrTiles; ++j) {
        // the stage kRrAhead ahead of this one, if the group has it: tile (j + kRrAhead) mod
        // kRrTiles of this chunk or of the next
        {
          const int jn = (j + kRrAhead) % kRrTiles;
          const int chn = ch + (j + kRrAhead) / kRrTiles;
          int buf_n = buf + kRrAhead;
          if (buf_n >= kRrStages) buf_n -= kRrStages;
          if (chn < n_chunks)
            issue(cidx[jn], chn, buf_n);
          else
            cp_async_commit();  // an empty group keeps the wait below uniform
        }
        if (one_run[j] && row0[j] != have_row) {
          const float4* d4 = reinterpret_cast<const float4*>(dst + (size_t)row0[j] * F +
                                                            (size_t)ch * kSdChunk);
#pragma unroll
          for (int q = 0; q < kSdChunk / 4; ++q) b[q] = __ldg(d4 + q);
          have_row = row0[j];
        }
        cp_async_wait<kRrAhead>();
        __syncwarp();
        const float4* s4 =
            reinterpret_cast<const float4*>(wbuf + buf * kRrStageFloats + lane * kSdPitch);
        if (one_run[j]) {
#pragma unroll
          for (int q = 0; q < kSdChunk / 4; ++q) {
            const float4 a = s4[q];
            acc[j] = combine<MSG, RED>(acc[j], a.x, b[q].x);
            acc[j] = combine<MSG, RED>(acc[j], a.y, b[q].y);
            acc[j] = combine<MSG, RED>(acc[j], a.z, b[q].z);
            acc[j] = combine<MSG, RED>(acc[j], a.w, b[q].w);
          }
        } else {
          const float4* d4 = reinterpret_cast<const float4*>(dst + (size_t)ridx[j] * F +
                                                            (size_t)ch * kSdChunk);
#pragma unroll
          for (int q = 0; q < kSdChunk / 4; ++q) {
            const float4 a = s4[q];
            const float4 d = __ldg(d4 + q);
            acc[j] = combine<MSG, RED>(acc[j], a.x, d.x);
            acc[j] = combine<MSG, RED>(acc[j], a.y, d.y);
            acc[j] = combine<MSG, RED>(acc[j], a.z, d.z);
            acc[j] = combine<MSG, RED>(acc[j], a.w, d.w);
          }
        }
        __syncwarp();  // every lane is done with this buffer before it is refilled
        if (++buf == kRrStages) buf = 0;
      }
    }
    cp_async_wait<0>();
#pragma unroll
    for (int j = 0; j < kRrTiles; ++j) {
      const long long e = (tile0 + g0 + j) * 32 + lane;
      if (e < nnz) out_store(out, (size_t)e, acc[j]);
    }
  }
  if (blockIdx.x == gridDim.x - 1 && warp == 0) wait_for_prior_grids();
}

// ---- the same tiles staged by the tensor memory accelerator -------------------------
//
// sddmm_tma_kernel: sddmm_tile_kernel's arithmetic with the gathers handed to TMA.  A stage's
// 32 src segments arrive as eight `cp.async.bulk.tensor.2d ... tile::gather4` copies (four
// arbitrary rows of the feature matrix x 32 floats each, issued by eight lanes), its dst
// segments as one or two more; the copies signal the stage's mbarrier with their byte
// count.  The tensor maps use the 128-byte swizzle, so the 16-byte piece q of the row at
// 128-byte slot r lies at piece q ^ (r & 7): lane l then reads ITS row with LDS.128 free of
// bank conflicts without the padded pitch, and the TMA unit writes whole lines where the
// sectors of a cp.async trickle into shared memory one by one.  Copies are asynchronous to
// the warp, so a ring of kTmStages stages per warp is really in flight.
//
// Every wait on an mbarrier is bounded: after `max_wait` clock cycles the warp records 1 in
// *status, stops issuing, waits (bounded again) for the copies it still has in flight and
// returns; the results of its remaining edges are then not written.
// Measured on B200 (114.6 M edges, feat_len 64; warps per CTA x stages per warp, warps per
// SM): 6 x 1, 36: 3.57 ms; 4 x 2, 20: 3.88; 6 x 2, 18: 4.00; 4 x 3, 12: 4.70; 4 x 4, 8: 7.60
// (sddmm_tile_kernel: 2.82).  More warps beat deeper rings here too, and every shape sits
// on the TMA unit's rate of about one four-row gather per 16 cycles and SM.
constexpr int kTmWarps = 6;
constexpr int kTmStages = 1;
constexpr int kTmMinCtas = 6;   // 36 warps per SM: at most 56 registers per thread
constexpr int kTmSrcBytes = 32 * 128;                 // 32 edges x 32 floats
constexpr int kTmDstBytes = kSdDstSlots * 128;        // up to 8 distinct dst rows
constexpr int kTmStageBytes = kTmSrcBytes + kTmDstBytes;
constexpr int kTmMetaInts = 32 + kSdDstSlots;         // per-lane words, slot rows
constexpr int kTmSmemBytes = 1024 + kTmWarps * kTmStages * (kTmStageBytes + 8 + 4 * kTmMetaInts);
constexpr long long kTmMaxWaitCycles = 4000000000LL;  // about two seconds
// how long one try_wait may keep the thread suspended (it wakes when the phase completes);
// without the hint the waiting warps poll, and their polls take issue slots
constexpr unsigned kTmSuspendNs = 2000;
static_assert(kTmStageBytes % 1024 == 0, "stages keep the swizzle's 1024-byte period");

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(kTmSuspendNs)
      : "memory");
  return ok != 0;
}
// Rows r0..r3 of the 2-D tensor behind `map`, 32 floats from column x (x * 4 is a multiple
// of 16 bytes: every chunk starts at a multiple of 32 floats), to 512 bytes at smem_dst.
__device__ __forceinline__ void tma_gather4(uint32_t smem_dst, const CUtensorMap* map, int x,
                                            int r0, int r1, int r2, int r3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(r0), "r"(r1), "r"(r2),
        "r"(r3), "r"(bar)
      : "memory");
}

template <int HEAD_DIM, int MSG, int RED>
__global__ void __launch_bounds__(kTmWarps * 32, kTmMinCtas)
sddmm_tma_kernel(const int* __restrict__ row, const int* __restrict__ col,
                 const __grid_constant__ CUtensorMap src_map,
                 const __grid_constant__ CUtensorMap dst_map, const float* __restrict__ dst,
                 const __grid_constant__ OutPtrs out, long long nnz, int F, int H,
                 int tiles_per_warp, int vec_heads, int* __restrict__ status,
                 long long max_wait) {
  constexpr unsigned kFull = 0xffffffffu;
  extern __shared__ unsigned char tm_smem[];
  launch_dependents();
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  const long long n_tiles = (nnz + 31) / 32;
  const long long tile0 = ((long long)blockIdx.x * kTmWarps + warp) * tiles_per_warp;
  if (tile0 >= n_tiles) return;  // (warp 0 of every CTA has tiles)
  const int my_tiles = (int)min((long long)tiles_per_warp, n_tiles - tile0);
  const int n_chunks = F / kSdChunk;
  const int total = my_tiles * n_chunks;
  const int chunks_per_head = HEAD_DIM == 0 ? (F / H) / kSdChunk : 1;

  // this warp's stages (1024-byte aligned), barriers and per-stage words
  const uint32_t raw = smem_u32(tm_smem);
  const uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  unsigned char* stages_gen = tm_smem + pad + (size_t)warp * kTmStages * kTmStageBytes;
  const uint32_t stages = raw + pad + warp * kTmStages * kTmStageBytes;
  const uint32_t bars = raw + pad + kTmWarps * kTmStages * kTmStageBytes + warp * kTmStages * 8;
  int* meta = reinterpret_cast<int*>(tm_smem + pad + kTmWarps * kTmStages * (kTmStageBytes + 8)) +
              warp * kTmStages * kTmMetaInts;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < kTmStages; ++s) mbar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();

  int r_iss = 0, c_iss = 0, word_iss = 0, n_slots = 1;
  bool head_iss = false;
  int r_ahead = 0, c_ahead = 0;
  auto fetch_indices = [&](int t) {
    const long long e = (tile0 + t) * 32 + lane;
    r_ahead = 0;
    c_ahead = 0;
    if (t < my_tiles && e < nnz) {
      r_ahead = ld_stream(row + e);
      c_ahead = ld_stream(col + e);
    }
  };
  auto begin_tile = [&](int t) {  // as in sddmm_tile_kernel
    r_iss = r_ahead;
    c_iss = c_ahead;
    fetch_indices(t + 1);
    const int r_left = __shfl_up_sync(kFull, r_iss, 1);
    head_iss = lane == 0 || r_iss != r_left;
    const unsigned run_heads = __ballot_sync(kFull, head_iss);
    n_slots = __popc(run_heads);
    const int slot = __popc(run_heads & (0xffffffffu >> (31 - lane))) - 1;
    word_iss = n_slots <= kSdDstSlots ? slot : -1 - r_iss;
  };
  int t_iss = 0, ch_iss = 0;
  auto issue = [&](int buf) {
    if (ch_iss == 0) begin_tile(t_iss);
    int* words = meta + buf * kTmMetaInts;
    int* slot_rows = words + 32;
    const bool staged = n_slots <= kSdDstSlots;
    words[lane] = word_iss;
    if (staged && head_iss) slot_rows[word_iss] = r_iss;
    const int n_dst = staged ? (n_slots > 4 ? 2 : 1) : 0;
    const uint32_t bar = bars + 8 * buf;
    if (lane == 0) mbar_arrive_expect_tx(bar, kTmSrcBytes + 512 * n_dst);
    // the lanes' reads of this buffer (generic proxy) come before the copies into it
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const int x = ch_iss * kSdChunk;
    const uint32_t sdst = stages + buf * kTmStageBytes;
    const int g = (lane & 7) * 4;
    const int c0 = __shfl_sync(kFull, c_iss, g), c1 = __shfl_sync(kFull, c_iss, g + 1);
    const int c2 = __shfl_sync(kFull, c_iss, g + 2), c3 = __shfl_sync(kFull, c_iss, g + 3);
    if (lane < 8) {
      tma_gather4(sdst + 512 * lane, &src_map, x, c0, c1, c2, c3, bar);
    } else if (lane < 8 + n_dst) {
      const int s0 = 4 * (lane - 8), last = n_slots - 1;
      tma_gather4(sdst + kTmSrcBytes + 512 * (lane - 8), &dst_map, x, slot_rows[min(s0, last)],
                  slot_rows[min(s0 + 1, last)], slot_rows[min(s0 + 2, last)],
                  slot_rows[min(s0 + 3, last)], bar);
    }
    if (++ch_iss == n_chunks) {
      ch_iss = 0;
      ++t_iss;
    }
  };
  auto wait_stage = [&](int buf, unsigned parity) -> bool {
    bool ok = mbar_try_wait(bars + 8 * buf, parity);
    if (!ok) {
      const long long t0 = clock64();
      do {
        ok = mbar_try_wait(bars + 8 * buf, parity);
      } while (!ok && clock64() - t0 < max_wait);
    }
    return __all_sync(kFull, ok);
  };

  fetch_indices(0);
  int issued = 0;
#pragma unroll
  for (int p = 0; p < kTmStages - 1; ++p)
    if (p < total) {
      issue(p);
      ++issued;
    }
  float acc = red_identity<RED>();
  int head = 0, chunk = 0, buf = 0, buf_issue = kTmStages - 1;
  unsigned parity = 0;
  long long e = tile0 * 32 + lane;
  float4 pend = make_float4(0.f, 0.f, 0.f, 0.f);
  auto finish_head = [&]() {  // as in sddmm_tile_kernel
    if (vec_heads) {
      switch (head & 3) {
        case 0: pend.x = acc; break;
        case 1: pend.y = acc; break;
        case 2: pend.z = acc; break;
        default:
          pend.w = acc;
          if (e < nnz) out_store(out, (size_t)e * H + head - 3, pend);
      }
    } else if (e < nnz) {
      out_store(out, (size_t)e * H + head, acc);
    }
    ++head;
    acc = red_identity<RED>();
  };
  int it = 0;
  bool gave_up = false;
  for (; it < total; ++it) {
    if (issued < total) {
      issue(buf_issue);
      ++issued;
    }
    if (!wait_stage(buf, parity)) {
      gave_up = true;
      break;
    }
    const unsigned char* stage = stages_gen + buf * kTmStageBytes;
    const int word = meta[buf * kTmMetaInts + lane];
    const unsigned char* srow = stage + lane * 128;
    const int sx = (lane & 7) << 4;
    const unsigned char* drow = stage + kTmSrcBytes + (word >= 0 ? word : 0) * 128;
    const int dx = word >= 0 ? (word & 7) << 4 : 0;
    const float4* dglob = reinterpret_cast<const float4*>(
        dst + (size_t)(word >= 0 ? 0 : -1 - word) * F + (size_t)chunk * kSdChunk);
#pragma unroll
    for (int q = 0; q < kSdChunk / 4; ++q) {
      const float4 a = *reinterpret_cast<const float4*>(srow + ((q << 4) ^ sx));
      const float4 b = word >= 0 ? *reinterpret_cast<const float4*>(drow + ((q << 4) ^ dx))
                                 : dglob[q];
      acc = combine<MSG, RED>(acc, a.x, b.x);
      acc = combine<MSG, RED>(acc, a.y, b.y);
      acc = combine<MSG, RED>(acc, a.z, b.z);
      acc = combine<MSG, RED>(acc, a.w, b.w);
      if (HEAD_DIM > 0 && ((q + 1) * 4) % (HEAD_DIM > 0 ? HEAD_DIM : 4) == 0) finish_head();
    }
    ++chunk;
    if (HEAD_DIM == 0 && chunk % chunks_per_head == 0) finish_head();
    if (chunk == n_chunks) {
      chunk = 0;
      head = 0;
      acc = red_identity<RED>();
      e += 32;
    }
    if (++buf == kTmStages) {
      buf = 0;
      parity ^= 1u;
    }
    buf_issue = buf_issue == kTmStages - 1 ? 0 : buf_issue + 1;
    __syncwarp();  // every lane is done with this buffer before it is refilled
  }
  if (gave_up) {
    if (lane == 0) atomicCAS(status, 0, 1);
    // the copies still in flight land in this CTA's shared memory: stay until they have
    // (bounded), starting with the stage that was being waited for
    for (int k = it; k < issued; ++k) {
      wait_stage(buf, parity);
      if (++buf == kTmStages) {
        buf = 0;
        parity ^= 1u;
      }
    }
  }
  if (blockIdx.x == gridDim.x - 1 && warp == 0) wait_for_prior_grids();
}

// Status word of the TMA kernel's bounded waits, one per GPU (fg_sddmm_status).
static __device__ int g_sddmm_status;

template <int MSG, int RED>
__global__ void __launch_bounds__(256)
sddmm_generic_kernel(const int* __restrict__ row, const int* __restrict__ col,
                     const float* __restrict__ src, const float* __restrict__ dst,
                     const __grid_constant__ OutPtrs out, long long n_out, int F, int H) {
  launch_dependents();
  if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) wait_for_prior_grids();  // thread 0 is valid
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= n_out) return;
  const long long e = i / H;
  const int h = (int)(i - e * H);
  const int D = F / H;
  const float* s = src + (size_t)col[e] * F + (size_t)h * D;
  const float* d = dst + (size_t)row[e] * F + (size_t)h * D;
  float acc = red_identity<RED>();
  for (int k = 0; k < D; ++k) acc = combine<MSG, RED>(acc, s[k], d[k]);
  out_store(out, (size_t)i, acc);
}

constexpr int kSdTilesPerWarp = kSdTilesPerWarpConst;

// -1 -> generic kernel; otherwise the HEAD_DIM template argument of the tile kernel.
static int sddmm_variant(int F, int H) {
  if (F % kSdChunk != 0 || F % H != 0) return -1;
  const int D = F / H;
  if (D % kSdChunk == 0) return D == kSdChunk ? kSdChunk : 0;
  if (D == 4 || D == 8 || (D == 16 && kSdChunk > 16)) return D;
  return -1;
}

// Copies n floats of this GPU's results into the same position of every peer's buffer
// (peer-mapped pointers): coalesced 16-byte loads and stores, a modest grid that leaves
// the SMs to the SDDMM kernel running beside it.  An alternative to storing the results
// to the peers from inside the SDDMM kernel, for callers whose slices of the peers'
// buffers are not 128-byte aligned (a warp's 32 results then straddle two lines of the
// peer's memory and the in-kernel stores leave a GPU at only ~360 GB/s; aligned, the
// in-kernel stores are the faster form: 0.67 against 1.01 ms per SDDMM on 8 GPUs).
template <bool VEC>
__global__ void __launch_bounds__(256)
sddmm_push_kernel(const float* __restrict__ src, const __grid_constant__ OutPtrs peers,
                  long long offset, long long n) {
  const long long stride = (long long)gridDim.x * 256;
  long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (VEC) {
    const long long n4 = n / 4;
    const float4* s4 = reinterpret_cast<const float4*>(src + offset);
    for (; i < n4; i += stride) {
      const float4 v = __ldcs(s4 + i);
      for (int q = 0; q < peers.n; ++q)
        __stcs(reinterpret_cast<float4*>(peers.p[q] + offset) + i, v);
    }
    i = n4 * 4 + ((long long)blockIdx.x * 256 + threadIdx.x);
    if (i < n) {
      const float v = src[offset + i];
      for (int q = 0; q < peers.n; ++q) peers.p[q][offset + i] = v;
    }
  } else {
    for (; i < n; i += stride) {
      const float v = __ldcs(src + offset + i);
      for (int q = 0; q < peers.n; ++q) peers.p[q][offset + i] = v;
    }
  }
}

constexpr int kPushMaxPieces = 8;
constexpr int kPushCtas = 64;
// One second stream and a set of events per device, made on first use and kept.
struct PushContext {
  cudaStream_t stream = nullptr;
  cudaEvent_t computed[kPushMaxPieces] = {nullptr};
  cudaEvent_t pushed = nullptr;
};
static PushContext* push_context(int device) {
  static thread_local PushContext ctx[64];
  if (device < 0 || device >= 64) return nullptr;
  PushContext* c = &ctx[device];
  if (!c->stream) {
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) return nullptr;
    for (int k = 0; k < kPushMaxPieces; ++k)
      if (cudaEventCreateWithFlags(&c->computed[k], cudaEventDisableTiming) != cudaSuccess)
        return nullptr;
    if (cudaEventCreateWithFlags(&c->pushed, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  }
  return c;
}

}  // namespace fg

extern "C" int fg_sddmm_num_launches(int64_t nnz, int32_t feat_len, int32_t num_heads) {
  (void)feat_len;
  (void)num_heads;
  return nnz > 0 ? 1 : 0;
}

extern "C" int fg_sddmm_describe(int64_t nnz, int32_t feat_len, int32_t num_heads, char* buf,
                                 int64_t buf_len) {
  using namespace fg;
  if (!buf || buf_len <= 0) return fail(FG_ERR_INVALID_ARGUMENT, "null buffer");
  if (num_heads <= 0 || feat_len <= 0 || feat_len % num_heads != 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "feat_len must be a positive multiple of num_heads");
  const int v = sddmm_variant(feat_len, num_heads);
  if (v < 0) {
    snprintf(buf, (size_t)buf_len,
             "sddmm_coo_f32 nnz=%lld feat_len=%d heads=%d | sddmm_generic_kernel grid=%lld x 256 thr",
             (long long)nnz, feat_len, num_heads,
             (long long)((nnz * num_heads + 255) / 256));
  } else {
    const long long tiles = (nnz + 31) / 32;
    const long long per_cta = (long long)kSdWarps * kSdTilesPerWarp;
    snprintf(buf, (size_t)buf_len,
             "sddmm_coo_f32 nnz=%lld feat_len=%d heads=%d | sddmm_tile_kernel<head_dim=%d> "
             "grid=%lld x %d thr, %d B smem, 32 edges x %d floats per stage, %d-stage ring per warp",
             (long long)nnz, feat_len, num_heads, v, (long long)((tiles + per_cta - 1) / per_cta),
             kSdWarps * 32, kSdSmemBytes, kSdChunk, kSdStages);
  }
  return FG_OK;
}

namespace fg {

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

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against
// libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of a row-major (rows x F) float matrix for tile::gather4 copies of 32-float
// row segments: a box of one row x 32 floats, 128-byte swizzle.
static bool make_segment_map(CUtensorMap* map, const float* base, int64_t rows, int32_t F) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || rows < 1) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)F, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)F * sizeof(float)};
  const cuuint32_t box[2] = {(cuuint32_t)kSdChunk, 1};
  const cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box,
            elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int* sddmm_status_word(int device) {
  static thread_local int* words[64] = {nullptr};
  if (device < 0 || device >= 64) return nullptr;
  if (!words[device]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sddmm_status) != cudaSuccess) return nullptr;
    words[device] = static_cast<int*>(p);
  }
  return words[device];
}

template <int MSG, int RED>
static cudaError_t sddmm_launch_kernels(int variant, long long grid, int tiles_per_warp,
                                        bool programmatic, const int32_t* row,
                                        const int32_t* col, const float* src, const float* dst,
                                        const OutPtrs& out, int64_t nnz, int64_t n_rows,
                                        int64_t n_cols, int32_t feat_len, int32_t num_heads,
                                        int32_t device, cudaStream_t st, bool tma,
                                        bool rowreg = false) {
  // heads leave four at a time where the lane's four results are one aligned 16-byte piece
  int vec_heads = num_heads % 4 == 0;
  for (int q = 0; q < out.n; ++q)
    if (reinterpret_cast<uintptr_t>(out.p[q]) % 16 != 0) vec_heads = 0;
  if (variant < 0)
    return launch_kernel(sddmm_generic_kernel<MSG, RED>, (unsigned)grid, 256, 0, st, programmatic,
                         row, col, src, dst, out, (long long)nnz * num_heads, feat_len, num_heads);
  if (rowreg) {
    static thread_local int configured_dev = -1;
    if (configured_dev != device) {
      cudaError_t e = cudaFuncSetAttribute(sddmm_rowreg_kernel<MSG, RED>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, kRrSmemBytes);
      if (e != cudaSuccess) return e;
      configured_dev = device;
    }
    return launch_kernel(sddmm_rowreg_kernel<MSG, RED>, (unsigned)grid, kRrWarps * 32, kRrSmemBytes,
                         st, programmatic, row, col, src, dst, out, (long long)nnz, feat_len,
                         tiles_per_warp);
  }
  if (tma && !(MSG == FG_MSG_MUL && RED == FG_REDUCE_SUM)) return cudaErrorNotSupported;
  if constexpr (MSG == FG_MSG_MUL && RED == FG_REDUCE_SUM) if (tma) {
    CUtensorMap src_map, dst_map;
    int* status = sddmm_status_word(device);
    if (!status || !make_segment_map(&src_map, src, n_cols, feat_len) ||
        !make_segment_map(&dst_map, dst, n_rows, feat_len))
      return cudaErrorInvalidValue;
#define FG_SD_LAUNCH_TMA(HPC)                                                                 \
  do {                                                                                        \
    static thread_local int configured_dev = -1;                                              \
    if (configured_dev != device) {                                                           \
      cudaError_t e__ = cudaFuncSetAttribute(sddmm_tma_kernel<HPC, MSG, RED>,                 \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                             kTmSmemBytes);                                   \
      if (e__ != cudaSuccess) return e__;                                                     \
      configured_dev = device;                                                                \
    }                                                                                         \
    cudaError_t l__ = launch_kernel(sddmm_tma_kernel<HPC, MSG, RED>, (unsigned)grid,          \
                                    kTmWarps * 32, kTmSmemBytes, st, programmatic, row, col,  \
                                    src_map, dst_map, dst, out, (long long)nnz, feat_len,     \
                                    num_heads, tiles_per_warp, vec_heads, status,             \
                                    kTmMaxWaitCycles);                                        \
    if (l__ != cudaSuccess) return l__;                                                       \
  } while (0)
    switch (variant) {
      case 0: FG_SD_LAUNCH_TMA(0); break;
      case 4: FG_SD_LAUNCH_TMA(4); break;
      case 8: FG_SD_LAUNCH_TMA(8); break;
      case 16: FG_SD_LAUNCH_TMA(16); break;
      default: FG_SD_LAUNCH_TMA(32); break;
    }
#undef FG_SD_LAUNCH_TMA
    return cudaGetLastError();
  }
#define FG_SD_LAUNCH(HPC)                                                                     \
  do {                                                                                        \
    static thread_local int configured_dev = -1;                                              \
    if (configured_dev != device) {                                                           \
      cudaError_t e__ = cudaFuncSetAttribute(sddmm_tile_kernel<HPC, MSG, RED>,                \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                             kSdSmemBytes);                                   \
      if (e__ != cudaSuccess) return e__;                                                     \
      configured_dev = device;                                                                \
    }                                                                                         \
    cudaError_t l__ = launch_kernel(sddmm_tile_kernel<HPC, MSG, RED>, (unsigned)grid,         \
                                    kSdWarps * 32, kSdSmemBytes, st, programmatic, row, col,  \
                                    src, dst, out, (long long)nnz, feat_len, num_heads,       \
                                    tiles_per_warp, vec_heads);                               \
    if (l__ != cudaSuccess) return l__;                                                       \
  } while (0)
  switch (variant) {
    case 0: FG_SD_LAUNCH(0); break;
    case 4: FG_SD_LAUNCH(4); break;
    case 8: FG_SD_LAUNCH(8); break;
    case 16: FG_SD_LAUNCH(16); break;
    default: FG_SD_LAUNCH(32); break;
  }
#undef FG_SD_LAUNCH
  return cudaGetLastError();
}

}  // namespace fg

static int sddmm_launch(const int32_t* row, const int32_t* col, const float* src,
                        const float* dst, float* const* outs, int32_t n_outs, int mcast,
                        int64_t nnz, int64_t n_rows, int64_t n_cols, int32_t feat_len,
                        int32_t num_heads, int32_t device, void* stream,
                        int32_t msg_op = FG_MSG_MUL, int32_t reduce_op = FG_REDUCE_SUM) {
  using namespace fg;
  const LaunchOptions opt = take_launch_options();
  if (msg_op < FG_MSG_MUL || msg_op > FG_MSG_COPY_RHS || reduce_op < FG_REDUCE_SUM ||
      reduce_op > FG_REDUCE_MIN)
    return fail(FG_ERR_INVALID_ARGUMENT, "unknown msg_op %d or reduce_op %d", (int)msg_op,
                (int)reduce_op);
  if (!outs || n_outs < 1 || n_outs > kMaxOutputs)
    return fail(FG_ERR_INVALID_ARGUMENT, "need 1 to %d output pointers, got %d", kMaxOutputs,
                (int)n_outs);
  OutPtrs out;
  out.n = n_outs;
  out.mcast = mcast;
  for (int q = 0; q < kMaxOutputs; ++q) out.p[q] = q < n_outs ? outs[q] : nullptr;
  if (nnz < 0 || n_rows < 0 || n_cols < 0 || feat_len <= 0 || num_heads <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad shape: nnz=%lld n_rows=%lld n_cols=%lld feat_len=%d heads=%d",
                (long long)nnz, (long long)n_rows, (long long)n_cols, (int)feat_len, (int)num_heads);
  if (feat_len % num_heads != 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "feat_len %d is not a multiple of num_heads %d",
                (int)feat_len, (int)num_heads);
  if (n_rows >= INT32_MAX || n_cols >= INT32_MAX)
    return fail(FG_ERR_UNSUPPORTED, "row/column counts must fit int32");
  if (nnz == 0) return FG_OK;
  if (!row || !col || !src || !dst) return fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  for (int q = 0; q < n_outs; ++q)
    if (!outs[q]) return fail(FG_ERR_INVALID_ARGUMENT, "output pointer %d is null", q);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));

  const bool aligned = (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                       (reinterpret_cast<uintptr_t>(dst) % 16 == 0);
  const int variant = aligned ? sddmm_variant(feat_len, num_heads) : -1;
  const bool tma = (opt.flags & FG_SDDMM_TMA_STAGING) != 0;
  if (tma && (variant < 0 || msg_op != FG_MSG_MUL || reduce_op != FG_REDUCE_SUM))
    return fail(FG_ERR_UNSUPPORTED, "FG_SDDMM_TMA_STAGING needs the multiply / sum operator pair, "
                "feat_len a multiple of 32 and 16-byte aligned feature arrays");
  const bool rowreg = (opt.flags & FG_SDDMM_ROW_REGISTERS) != 0 && variant >= 0 &&
                      num_heads == 1 && !tma;
  const int warps = tma ? kTmWarps : rowreg ? kRrWarps : kSdWarps;
  long long grid;
  long long tiles_per_warp = kSdTilesPerWarp;
  if (variant < 0) {
    grid = ((long long)nnz * num_heads + 255) / 256;
    if (grid >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "output too large for the generic kernel");
  } else {
    const long long tiles = (nnz + 31) / 32;
    // a bounded grid (max_ctas): every warp walks a longer stretch of the edge list
    if (opt.max_ctas > 0)
      tiles_per_warp = std::max<long long>(
          tiles_per_warp, (tiles + (long long)warps * opt.max_ctas - 1) / ((long long)warps * opt.max_ctas));
    if (rowreg) tiles_per_warp = (tiles_per_warp + kRrTiles - 1) / kRrTiles * kRrTiles;
    if (tiles_per_warp >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "edge count too large");
    const long long per_cta = (long long)warps * tiles_per_warp;
    grid = (tiles + per_cta - 1) / per_cta;
    if (grid >= INT32_MAX) return fail(FG_ERR_UNSUPPORTED, "edge count too large");
  }
  const bool programmatic = (opt.flags & FG_LAUNCH_PROGRAMMATIC) != 0;
  cudaError_t err = cudaSuccess;
#define FG_SD_OPS(M, R)                                                                          \
  err = sddmm_launch_kernels<M, R>(variant, grid, (int)tiles_per_warp, programmatic, row, col,  \
                                   src, dst, out, nnz, n_rows, n_cols, feat_len, num_heads,     \
                                   device, st, tma, rowreg)
  FG_DISPATCH_OPS(msg_op, reduce_op, FG_SD_OPS);
#undef FG_SD_OPS
  FG_CUDA_TRY(err);
  return FG_OK;
}

extern "C" int fg_sddmm_status(int32_t device, int32_t* device_status) {
  using namespace fg;
  if (!device_status) return fail(FG_ERR_INVALID_ARGUMENT, "device_status is null");
  *device_status = 0;
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  int* word = sddmm_status_word(device);
  if (!word) return fail(FG_ERR_CUDA, "cannot find the status word");
  FG_CUDA_TRY(cudaDeviceSynchronize());
  int v = 0;
  FG_CUDA_TRY(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost));
  *device_status = v;
  if (v != 0) {
    // reported once: the word is cleared so that later calls are judged on their own
    FG_CUDA_TRY(cudaMemset(word, 0, sizeof(int)));
    return fail(FG_ERR_CUDA, "sddmm_tma_kernel: a bounded wait for a TMA copy gave up; the "
                "results of the edges behind it were not written");
  }
  return FG_OK;
}

extern "C" int fg_sddmm_coo_f32_general(const int32_t* row, const int32_t* col, const float* src,
                                        const float* dst, float* out, int64_t nnz,
                                        int64_t n_rows, int64_t n_cols, int32_t feat_len,
                                        int32_t num_heads, int32_t msg_op, int32_t reduce_op,
                                        int32_t device, void* stream) {
  if (nnz > 0 && !out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  float* outs[1] = {out};
  return sddmm_launch(row, col, src, dst, outs, 1, 0, nnz, n_rows, n_cols, feat_len, num_heads,
                      device, stream, msg_op, reduce_op);
}

extern "C" int fg_sddmm_coo_f32_multi(const int32_t* row, const int32_t* col, const float* src,
                                      const float* dst, float* const* outs, int32_t n_outs,
                                      int64_t nnz, int64_t n_rows, int64_t n_cols,
                                      int32_t feat_len, int32_t num_heads, int32_t device,
                                      void* stream) {
  return sddmm_launch(row, col, src, dst, outs, n_outs, 0, nnz, n_rows, n_cols, feat_len,
                      num_heads, device, stream);
}

extern "C" int fg_sddmm_coo_f32_mcast(const int32_t* row, const int32_t* col, const float* src,
                                      const float* dst, float* out_mcast, int64_t nnz,
                                      int64_t n_rows, int64_t n_cols, int32_t feat_len,
                                      int32_t num_heads, int32_t device, void* stream) {
  if (nnz > 0 && !out_mcast) return fg::fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  float* outs[1] = {out_mcast};
  return sddmm_launch(row, col, src, dst, outs, 1, 1, nnz, n_rows, n_cols, feat_len, num_heads,
                      device, stream);
}

extern "C" int fg_sddmm_coo_f32(const int32_t* row, const int32_t* col, const float* src,
                                const float* dst, float* out, int64_t nnz, int64_t n_rows,
                                int64_t n_cols, int32_t feat_len, int32_t num_heads,
                                int32_t device, void* stream) {
  if (nnz > 0 && !out) return fg::fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  float* outs[1] = {out};
  return fg_sddmm_coo_f32_multi(row, col, src, dst, nnz > 0 ? outs : outs, 1, nnz, n_rows, n_cols,
                                feat_len, num_heads, device, stream);
}

extern "C" int fg_sddmm_coo_f32_host(const int32_t* row, const int32_t* col,
                                     const float* src_host, const float* dst_host,
                                     float* out_host, float* src_stage, float* dst_stage,
                                     float* out_stage, int64_t nnz, int64_t n_rows,
                                     int64_t n_cols, int32_t feat_len, int32_t num_heads,
                                     int32_t device, void* stream) {
  using namespace fg;
  // the options of this call go to every piece's kernel (but for the programmatic launch:
  // the pieces follow copies)
  LaunchOptions opt = take_launch_options();
  opt.flags &= ~FG_LAUNCH_PROGRAMMATIC;
  if (!src_host || !dst_host || !out_host || !src_stage || !dst_stage || !out_stage)
    return fail(FG_ERR_INVALID_ARGUMENT, "null host or staging buffer");
  if (nnz < 0 || n_rows < 0 || n_cols < 0 || feat_len <= 0 || num_heads <= 0)
    return fail(FG_ERR_INVALID_ARGUMENT, "bad shape");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  const size_t sb = sizeof(float) * (size_t)n_cols * feat_len;
  const size_t db = sizeof(float) * (size_t)n_rows * feat_len;
  if (sb) FG_CUDA_TRY(cudaMemcpyAsync(src_stage, src_host, sb, cudaMemcpyHostToDevice, st));
  if (db) FG_CUDA_TRY(cudaMemcpyAsync(dst_stage, dst_host, db, cudaMemcpyHostToDevice, st));
  // The output (4 bytes per edge and head) dominates the transfers, so the edge list is
  // cut into pieces: while piece k+1 is computed, piece k travels to the host on a second
  // stream.  Small inputs take one piece.
  const int pieces = nnz >= (1 << 22) ? kPushMaxPieces : 1;
  // the second stream and its events are made once per device and host thread, and kept
  PushContext* pc = pieces > 1 ? push_context(device) : nullptr;
  if (pieces > 1 && !pc) return fail(FG_ERR_CUDA, "cannot create the copy stream or its events");
  int rc = FG_OK;
  cudaError_t err = cudaSuccess;
  for (int k = 0; k < pieces && rc == FG_OK && err == cudaSuccess; ++k) {
    const int64_t e0 = nnz * k / pieces, e1 = nnz * (k + 1) / pieces;
    if (e1 == e0) continue;
    if (opt.flags || opt.max_ctas) fg_next_launch_options(opt.flags, opt.max_ctas);
    rc = fg_sddmm_coo_f32(row + e0, col + e0, src_stage, dst_stage, out_stage + e0 * num_heads,
                          e1 - e0, n_rows, n_cols, feat_len, num_heads, device, stream);
    if (rc != FG_OK) break;
    const size_t bytes = sizeof(float) * (size_t)(e1 - e0) * num_heads;
    if (pc) {
      err = cudaEventRecord(pc->computed[k], st);
      if (err == cudaSuccess) err = cudaStreamWaitEvent(pc->stream, pc->computed[k], 0);
      if (err == cudaSuccess)
        err = cudaMemcpyAsync(out_host + e0 * num_heads, out_stage + e0 * num_heads, bytes,
                              cudaMemcpyDeviceToHost, pc->stream);
    } else {
      err = cudaMemcpyAsync(out_host + e0 * num_heads, out_stage + e0 * num_heads, bytes,
                            cudaMemcpyDeviceToHost, st);
    }
  }
  // both streams are drained also after a failure: no copy of this call outlives it
  const cudaError_t e1 = cudaStreamSynchronize(st);
  const cudaError_t e2 = pc ? cudaStreamSynchronize(pc->stream) : cudaSuccess;
  if (err == cudaSuccess) err = e1 != cudaSuccess ? e1 : e2;
  if (rc != FG_OK) return rc;
  if (err != cudaSuccess)
    return fail(FG_ERR_CUDA, "fg_sddmm_coo_f32_host: %s", cudaGetErrorString(err));
  return FG_OK;
}

extern "C" int fg_sddmm_coo_f32_push(const int32_t* row, const int32_t* col, const float* src,
                                     const float* dst, float* out, float* const* peer_outs,
                                     int32_t n_peers, int64_t nnz, int64_t n_rows, int64_t n_cols,
                                     int32_t feat_len, int32_t num_heads, int32_t device,
                                     void* stream) {
  using namespace fg;
  if (n_peers < 0 || n_peers > kMaxOutputs || (n_peers > 0 && !peer_outs))
    return fail(FG_ERR_INVALID_ARGUMENT, "need 0 to %d peer pointers, got %d", kMaxOutputs,
                (int)n_peers);
  if (n_peers == 0 || nnz <= 0)
    return fg_sddmm_coo_f32(row, col, src, dst, out, nnz, n_rows, n_cols, feat_len, num_heads,
                            device, stream);
  LaunchOptions opt = take_launch_options();  // handed to every piece's kernel
  opt.flags &= ~FG_LAUNCH_PROGRAMMATIC;
  if (!out) return fail(FG_ERR_INVALID_ARGUMENT, "null device pointer");
  OutPtrs peers;
  peers.n = n_peers;
  peers.mcast = 0;
  bool vec = reinterpret_cast<uintptr_t>(out) % 16 == 0;
  for (int q = 0; q < kMaxOutputs; ++q) {
    peers.p[q] = q < n_peers ? peer_outs[q] : nullptr;
    if (q < n_peers && !peer_outs[q])
      return fail(FG_ERR_INVALID_ARGUMENT, "peer pointer %d is null", q);
    if (q < n_peers && reinterpret_cast<uintptr_t>(peer_outs[q]) % 16 != 0) vec = false;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  DeviceGuard guard(device);
  if (guard.status != cudaSuccess)
    return fail(FG_ERR_CUDA, "cannot select device %d: %s", device,
                cudaGetErrorString(guard.status));
  PushContext* pc = push_context(device);
  if (!pc) return fail(FG_ERR_CUDA, "cannot create the push stream or its events");
  // Pieces of whole 32-edge tiles: piece k is pushed to the peers while piece k+1 computes.
  const int pieces = nnz >= (1 << 20) ? 4 : 1;
  const int64_t tiles = (nnz + 31) / 32;
  for (int k = 0; k < pieces; ++k) {
    const int64_t e0 = std::min<int64_t>(nnz, tiles * k / pieces * 32);
    const int64_t e1 = std::min<int64_t>(nnz, tiles * (k + 1) / pieces * 32);
    if (e1 <= e0) continue;
    if (opt.flags || opt.max_ctas) fg_next_launch_options(opt.flags, opt.max_ctas);
    const int rc = fg_sddmm_coo_f32(row + e0, col + e0, src, dst, out + e0 * num_heads, e1 - e0,
                                    n_rows, n_cols, feat_len, num_heads, device, stream);
    if (rc != FG_OK) return rc;
    FG_CUDA_TRY(cudaEventRecord(pc->computed[k], st));
    FG_CUDA_TRY(cudaStreamWaitEvent(pc->stream, pc->computed[k], 0));
    const long long off = (long long)e0 * num_heads, n = (long long)(e1 - e0) * num_heads;
    if (vec)
      sddmm_push_kernel<true><<<kPushCtas, 256, 0, pc->stream>>>(out, peers, off, n);
    else
      sddmm_push_kernel<false><<<kPushCtas, 256, 0, pc->stream>>>(out, peers, off, n);
    FG_CUDA_TRY(cudaGetLastError());
  }
  FG_CUDA_TRY(cudaEventRecord(pc->pushed, pc->stream));
  FG_CUDA_TRY(cudaStreamWaitEvent(st, pc->pushed, 0));
  return FG_OK;
}
