// Grouped GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue.
//
// One persistent CTA per SM (or a cluster of two CTAs per 256-row tile in pair mode), eight warps:
//   warp 0      TMA producer (one lane issues cp.async.bulk.tensor loads)
//   warp 1      TMEM allocator and MMA issuer (one lane issues tcgen05.mma)
//   warps 2..5  epilogue: tcgen05.ld the accumulator, convert, stage, store
//   warps 6..7  ragged rows: dispatch warps of a fused launch (push this rank's rows to their
//               owners while the GEMM consumes the experts whose rows have arrived);
//               ragged reduction, single CTA: warp 6 clears the rows past a group's end in the
//               group's last k-block, warp 7 is a second MMA issuer (tiles alternate)
// A ring of shared-memory stages feeds the tensor core; two 128x256 fp32 accumulators in TMEM
// let the epilogue of tile i overlap the main loop of tile i+1.
//
// Two problem kinds share the kernel:
//   kGroupedRows  out[rows of group g, :] = A[rows of g, 0:K] * B_g      (ragged M)
//       used for FC1, FC2 and the two input-gradient GEMMs
//   kGroupedReduce out_g[m', n'] = sum over rows of g: A[row, m'] * B[row, n'] (ragged K)
//       used for the two weight-gradient GEMMs; both operands are MN-major
#pragma once

#include "common.cuh"

namespace mm {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;
constexpr int kUmmaK = 16;
constexpr int kStages = 4;                                        // one CTA per tile
constexpr int kStageABytes = kBlockM * kBlockK * 2;               // 16 KB
constexpr int kStageBBytes = kBlockN * kBlockK * 2;               // 32 KB
constexpr int kStageBytes = kStageABytes + kStageBBytes;          // 48 KB
// Pair mode (cta_group::2): two CTAs of a cluster share one 256x256 tile; each loads its own
// 128 rows of A and half of B (128 columns), so a stage is 32 KB and six stages fit.
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kStageABytes + kStageBBytes / 2;  // 32 KB
constexpr int kMaxStages = 6;
constexpr int kBoxBytes = 64 * 64 * 2;                            // one 64x64 MN-major box
constexpr int kEpiWarps = 4;
constexpr int kStagingPerWarp = 2 * 32 * 128;                     // two 32-row x 128-byte buffers
constexpr int kDispatchWarps = 2;                                  // row-push warps of a fused launch
constexpr int kGemmThreads = 32 * (2 + kEpiWarps + kDispatchWarps);
constexpr int kTmemCols = 512;
constexpr int kGemmSmemBytes =
    kStages * kStageBytes + kEpiWarps * kStagingPerWarp + 256 /*barriers*/ + 1024 /*alignment*/;

enum GemmKind : int32_t { kGroupedRows = 0, kGroupedReduce = 1 };
enum EpiMode : int32_t { kEpiStore = 0, kEpiSwiglu = 1, kEpiScatter = 2 };
enum Activation : int32_t { kActSwiglu = 0, kActSitu = 1, kActClampSwiglu = 2 };

struct GemmParams {
  int32_t kind;
  int32_t epi;
  int32_t num_groups;
  int32_t N;             // logical output columns (kEpiSwiglu: F; kGroupedReduce: n' extent)
  int32_t K;             // reduction extent (kGroupedRows)
  int32_t Mw;            // kGroupedReduce: m' extent
  int32_t a_mn;          // A operand is MN-major
  int32_t b_mn;          // B operand is MN-major
  int32_t n_tiles;       // tiles along N (kEpiSwiglu: F / 128)
  int32_t m_tiles;       // kGroupedReduce: tiles along m'
  int32_t swiglu_F;      // column offset of the "up" half inside B and inside out2
  int32_t tma_store;     // kGroupedReduce: output tiles leave through TMA tensor stores
  int32_t wide_store;    // row stores in 256-byte pieces (scatter over NVLink)
  int32_t pair;          // 1: cta_group::2, clusters of two CTAs, 256-row tiles
  int32_t prefetch_kb;   // skinny kernel: k-blocks of weights requested into L2 ahead of the loads
  int32_t unit_walk;     // single-CTA ragged reduction: walk whole units (see TileCursor)
  // MN-major operands are 64x64 boxes in shared memory.  When the operand's extent allows it
  // the tensor map carries the box index as an extra dimension, so that one TMA instruction
  // brings all boxes of a stage (the producer lane is bound by the number of instructions):
  int32_t a_multibox;    // kGroupedReduce: tmA is {64, rows, Mw / 64}, box {64, 64, 2}
  int32_t b_multibox;    // 1: tmB is {64, k, cols / 64, groups}, box {64, 64, boxes, 1}
                         // 2: fused FC1, one CTA: {64, k, F / 64, 2, groups}, box {64, 64, 2, 2, 1}
  int32_t act;
  float act_beta;
  float act_linear_beta; // <= 0: no transform on up
  float act_clamp;
  uint32_t idesc;
  const int32_t* group_offs;    // [num_groups + 1] row offsets of each group
  const int32_t* mtile_group;   // kGroupedRows: group of each 128-row tile
  const int32_t* mtile_row0;    // kGroupedRows: first row of each 128-row tile
  const int32_t* num_mtiles;    // kGroupedRows: device scalar, number of 128-row tiles
  __nv_bfloat16* out;
  int64_t ld_out;
  int64_t out_group_stride;     // kGroupedReduce: elements between consecutive groups
  __nv_bfloat16* out2;          // kEpiSwiglu: raw gate|up rows, may be null
  int64_t ld_out2;
  const float* row_weight;      // kEpiSwiglu: fp32 weight of each row
  __nv_bfloat16* row_weight_bf16;  // kEpiSwiglu: bf16 copy of the row weights (out), may be null
  const int32_t* row_dst_rank;  // kEpiScatter: destination rank of each row
  const int32_t* row_dst_pos;   // kEpiScatter: destination row index
  __nv_bfloat16* const* peer_bases;  // kEpiScatter: base pointer of the destination buffer per rank
  int64_t ld_dst;
  StatusRecord* status;
  // ---- fused dispatch (FC1 and the FC2 input gradient): two extra warps per CTA push this
  // rank's send rows into the owning ranks' receive buffers while the GEMM roles consume the
  // experts whose rows have arrived.  disp_src == nullptr: plain GEMM on resident rows.
  const uint8_t* disp_src;            // [tokens, row_bytes] rows to send
  int32_t disp_row_bytes;
  int32_t disp_rank, disp_world, disp_epr, disp_capacity, disp_epoch;
  const float* disp_weights;          // per-route fp32 weight sent alongside, may be null
  const int32_t* disp_send_token;     // send row -> token
  const int32_t* disp_send_route;     // send row -> flat route
  const int32_t* disp_bucket_starts;  // first send row of each bucket
  const int32_t* disp_dst_starts;     // first destination row of each bucket
  const int32_t* disp_counts;         // rows per bucket (local count row)
  const int32_t* disp_order_prefix;   // [buckets + 1] prefix of the counts in dispatch order
  const int32_t* disp_num_send;       // device scalar: number of send rows
  int32_t* disp_bucket_done;          // [buckets] rows delivered so far: zero at launch, and zero
                                      // again once a bucket is complete
  void* const* disp_peer_rows;        // receive buffer base per rank
  float* const* disp_peer_weights;    // routing-weight buffer base per rank
  int32_t* const* disp_peer_flags;    // arrival flags base per rank: [world * epr] per rank
  const int32_t* disp_my_flags;       // this rank's arrival flags
  // MM_PROFILE builds only: [grid, 16] clock counters of the roles' waits (see prof_now)
  unsigned long long* prof;
  int32_t prof_skip_mma;   // MM_PROFILE builds only: stages are freed without issuing MMAs
};

// Wait-time accounting of an instrumented build (-DMM_PROFILE): each role sums the SM clocks it
// spends in its waits and writes them out when it leaves.  Without the macro the helpers fold
// to constants and the counters disappear.
__device__ __forceinline__ long long prof_now() {
#ifdef MM_PROFILE
  return clock64();
#else
  return 0;
#endif
}
__device__ __forceinline__ void prof_store(const GemmParams& p, int slot, long long v) {
#ifdef MM_PROFILE
  if (p.prof != nullptr) p.prof[(size_t)blockIdx.x * 16 + slot] = (unsigned long long)v;
#endif
}

__device__ __forceinline__ int32_t total_tiles(const GemmParams& p) {
  if (p.kind == kGroupedRows) return (*p.num_mtiles) * p.n_tiles;
  return p.num_groups * p.m_tiles * p.n_tiles;
}

// Tile t of the launch as seen by CTA `cta_rank` of its pair (always 0 without pairing).
// A tile spans 128 rows, or 256 in pair mode with 128 rows per CTA.
__device__ __forceinline__ TileInfo decode_tile(const GemmParams& p, int32_t t, int32_t cta_rank) {
  TileInfo ti;
  const int32_t shift = p.pair ? 8 : 7;
  const int32_t tile_rows = 1 << shift;
  if (p.kind == kGroupedRows) {
    // Group-major order: all tiles of one expert are consecutive (n-tile outer, row tile
    // inner), so the CTAs running at the same time share one expert's rows and weights in L2.
    // Tile t lies in the group of row tile t / n_tiles because group g owns the tile
    // range [first_g * n_tiles, (first_g + cnt_g) * n_tiles).
    const int32_t u = t / p.n_tiles;
    ti.group = p.mtile_group[u];
    const int32_t g0 = p.group_offs[ti.group];
    const int32_t end = p.group_offs[ti.group + 1];
    const int32_t first = u - ((p.mtile_row0[u] - g0) >> shift);
    const int32_t cnt = (end - g0 + tile_rows - 1) >> shift;
    const int32_t local = t - first * p.n_tiles;
    const int32_t nt = local / cnt;
    const int32_t mj = local - nt * cnt;
    ti.row0 = g0 + mj * tile_rows + cta_rank * kBlockM;
    ti.rows_valid = max(0, min(kBlockM, end - ti.row0));
    ti.n0 = nt * (p.epi == kEpiSwiglu ? kBlockN / 2 : kBlockN);
    ti.num_kb = (p.K + kBlockK - 1) / kBlockK;
    ti.krow0 = 0;
    ti.kcnt = 0;
  } else {
    const int32_t per_group = p.m_tiles * p.n_tiles;
    ti.group = t / per_group;
    const int32_t r = t - ti.group * per_group;
    const int32_t nt = r / p.m_tiles;
    const int32_t mt = r - nt * p.m_tiles;
    ti.row0 = mt * tile_rows + cta_rank * kBlockM;
    ti.rows_valid = max(0, min(kBlockM, p.Mw - ti.row0));
    ti.n0 = nt * kBlockN;
    ti.krow0 = p.group_offs[ti.group];
    ti.kcnt = p.group_offs[ti.group + 1] - ti.krow0;
    ti.num_kb = (ti.kcnt + kBlockK - 1) / kBlockK;
  }
  return ti;
}

__device__ __forceinline__ float gated_activation(float g, float u, const GemmParams& p) {
  if (p.act == kActSwiglu) {
    return g / (1.0f + __expf(-g)) * u;
  } else if (p.act == kActClampSwiglu) {
    g = fminf(g, p.act_clamp);
    u = fminf(fmaxf(u, -p.act_clamp), p.act_clamp);
    return g / (1.0f + __expf(-g)) * u;
  } else {
    const float a = p.act_beta * tanhf(g / p.act_beta) / (1.0f + __expf(-g));
    if (p.act_linear_beta > 0.0f) u = p.act_linear_beta * tanhf(u / p.act_linear_beta);
    return a * u;
  }
}

// Staging buffers hold 32 rows x 128 bytes (64 bf16 columns); the 16-byte chunk c of row r
// lives at r * 128 + ((c ^ (r & 7)) << 4).  That is the 128-byte TMA swizzle, so a buffer can
// leave through a tensor store, and it keeps both the row-wise writes and the chunk-wise
// reads free of bank conflicts.

// Write 32 bf16 values (chunks first_chunk .. first_chunk + 3) of this lane's row.
__device__ __forceinline__ void stage_half_row(uint8_t* stg, uint32_t lane, int first_chunk,
                                               const uint32_t (&v)[16]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q = make_uint4(v[4 * c + 0], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)(first_chunk + c)) ^ (lane & 7)) << 4)) = q;
  }
}

// Convert 64 fp32 accumulator values of this lane's row to bf16 and stage them.
__device__ __forceinline__ void stage_row_f32(uint8_t* stg, uint32_t lane, const uint32_t (&r)[64]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]), __uint_as_float(r[8 * c + 1]));
    q.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]));
    q.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]));
    q.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]));
    *reinterpret_cast<uint4*>(stg + lane * 128 + ((((uint32_t)c) ^ (lane & 7)) << 4)) = q;
  }
}

// Store a staged 32-row x 64-column bf16 block with plain stores: each warp instruction
// writes 4 rows x 128 bytes.  row_ptr is this lane's row base (already offset to the block's
// first column); cols_valid masks the columns past the logical output width.
__device__ __forceinline__ void flush_rows(const uint8_t* stg, uint32_t lane, uint8_t* row_ptr,
                                           int valid, int cols_valid) {
  const uint32_t c = lane & 7;
  const bool col_ok = (int)(c * 8) < cols_valid;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const uint32_t r = it * 4 + (lane >> 3);
    const uint4 q = *reinterpret_cast<const uint4*>(stg + r * 128 + ((c ^ (r & 7)) << 4));
    const uint64_t pr = __shfl_sync(0xffffffffu, (unsigned long long)row_ptr, r);
    const int ok = __shfl_sync(0xffffffffu, valid, r);
    if (ok && col_ok) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pr) + c * 16) = q;
  }
}

// Wide variant: the warp's whole 8 KB staging area holds 32 rows x 256 bytes (128 columns),
// chunk cc of row r at r * 256 + ((cc ^ (r & 15)) << 4); a warp instruction then writes
// 2 rows x 256 contiguous bytes, which suits stores that cross NVLink.
__device__ __forceinline__ void stage_row_f32_wide(uint8_t* stg, uint32_t lane, int half,
                                                   const uint32_t (&r)[64]) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = pack_bf16x2(__uint_as_float(r[8 * c + 0]), __uint_as_float(r[8 * c + 1]));
    q.y = pack_bf16x2(__uint_as_float(r[8 * c + 2]), __uint_as_float(r[8 * c + 3]));
    q.z = pack_bf16x2(__uint_as_float(r[8 * c + 4]), __uint_as_float(r[8 * c + 5]));
    q.w = pack_bf16x2(__uint_as_float(r[8 * c + 6]), __uint_as_float(r[8 * c + 7]));
    const uint32_t cc = (uint32_t)(half * 8 + c);
    *reinterpret_cast<uint4*>(stg + lane * 256 + ((cc ^ (lane & 15)) << 4)) = q;
  }
}

__device__ __forceinline__ void flush_rows_wide(const uint8_t* stg, uint32_t lane,
                                                uint8_t* row_ptr, int valid, int cols_valid) {
  const uint32_t cc = lane & 15;
  const bool col_ok = (int)(cc * 8) < cols_valid;
#pragma unroll
  for (int it = 0; it < 16; ++it) {
    const uint32_t r = it * 2 + (lane >> 4);
    const uint4 q = *reinterpret_cast<const uint4*>(stg + r * 256 + ((cc ^ (r & 15)) << 4));
    const uint64_t pr = __shfl_sync(0xffffffffu, (unsigned long long)row_ptr, r);
    const int ok = __shfl_sync(0xffffffffu, valid, r);
    if (ok && col_ok) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(pr) + cc * 16) = q;
  }
}

template <bool kPair>
__device__ __forceinline__ void load2d(bool direct, void* dst, const CUtensorMap* map,
                                       uint64_t* bar, int32_t c0, int32_t c1) {
  if constexpr (kPair) {
    if (direct) {
      tma_load_2d_pair(dst, map, bar, c0, c1);
      return;
    }
  }
  tma_load_2d(dst, map, bar, c0, c1);
}

template <bool kPair>
__device__ __forceinline__ void load4d(bool direct, void* dst, const CUtensorMap* map,
                                       uint64_t* bar, int32_t c0, int32_t c1, int32_t c2,
                                       int32_t c3) {
  if constexpr (kPair) {
    if (direct) {
      tma_load_4d_pair(dst, map, bar, c0, c1, c2, c3);
      return;
    }
  }
  tma_load_4d(dst, map, bar, c0, c1, c2, c3);
}

template <bool kPair>
__device__ __forceinline__ void load3d(bool direct, void* dst, const CUtensorMap* map,
                                       uint64_t* bar, int32_t c0, int32_t c1, int32_t c2) {
  if constexpr (kPair) {
    if (direct) {
      tma_load_3d_pair(dst, map, bar, c0, c1, c2);
      return;
    }
  }
  tma_load_3d(dst, map, bar, c0, c1, c2);
}

// Body of one dispatch warp of a fused launch: push this rank's send rows into the owning
// ranks' receive buffers in dispatch order, count delivered rows per (destination, expert)
// bucket and flag a bucket's arrival at the destination once it is complete.  Never waits.
//
// A warp works in batches of kDispatchBatchRows consecutive rows of the dispatch order.  Lane r
// (r < batch rows) owns row r of the batch: it keeps the row's source and destination
// pointers, and the warp copies the rows in 7 KB segments through two register buffers, so the
// loads of one segment are in flight while the previous one is stored.  The lookups of the
// next batch are issued before the fence of the current one and overlap its draining stores.
constexpr int kDispatchBatchRows = 8;
constexpr int kDispatchSegChunks = 14;   // 16-byte chunks per lane and segment

struct DispatchRow {       // held by lane r for row r of a batch
  const uint8_t* src;      // nullptr: nothing to copy (past the end, or receive overflow)
  uint8_t* dst;
  int32_t bucket;          // -1: no row
  int32_t dst_rank;
};

// Position of dispatch-order index j: the largest q with order_prefix[q] <= j (empty buckets
// share their successor's prefix).  All lanes take part; two 32-way steps cover 1024 buckets,
// a third 32 768.
__device__ __forceinline__ int32_t dispatch_find_bucket(const int32_t* __restrict__ prefix,
                                                        int32_t nb, int32_t j, uint32_t lane) {
  int32_t lo = 0, span = nb;          // the answer lies in [lo, lo + span)
  while (span > 1) {
    const int32_t step = (span + 31) >> 5;
    const int32_t off = (int32_t)lane * step;
    const bool le = off < span && prefix[lo + off] <= j;
    const uint32_t m = __ballot_sync(0xffffffffu, le);
    const int32_t seg = 31 - __clz((int)m);        // lane 0 always qualifies: prefix[lo] <= j
    lo += seg * step;
    span = min(step, span - seg * step);
  }
  return lo;
}

__device__ __forceinline__ DispatchRow dispatch_resolve(const GemmParams& p, int32_t j0,
                                                        int32_t n_send, int32_t nb, uint32_t lane) {
  DispatchRow row;
  row.src = nullptr;
  row.dst = nullptr;
  row.bucket = -1;
  row.dst_rank = 0;
  if (j0 >= n_send) return row;
  int32_t q = dispatch_find_bucket(p.disp_order_prefix, nb, j0, lane);
  const int32_t j = j0 + (int32_t)lane;
  if ((int32_t)lane < kDispatchBatchRows && j < n_send) {
    // the rows after the first lie in the same bucket or a few buckets further on
    while (q + 1 < nb && p.disp_order_prefix[q + 1] <= j) ++q;
    const int32_t b = dispatch_order_bucket(q, p.disp_rank, p.disp_world, p.disp_epr);
    const int32_t in_bucket = j - p.disp_order_prefix[q];
    const int32_t i = p.disp_bucket_starts[b] + in_bucket;
    const int32_t dst_row = p.disp_dst_starts[b] + in_bucket;
    row.bucket = b;
    row.dst_rank = b / p.disp_epr;
    if (dst_row < p.disp_capacity) {     // overflow: the metadata kernel reports it
      row.src = p.disp_src + (size_t)p.disp_send_token[i] * p.disp_row_bytes;
      row.dst = reinterpret_cast<uint8_t*>(p.disp_peer_rows[row.dst_rank]) +
                (size_t)dst_row * p.disp_row_bytes;
      if (p.disp_weights != nullptr)
        p.disp_peer_weights[row.dst_rank][dst_row] = p.disp_weights[p.disp_send_route[i]];
    }
  }
  return row;
}

__device__ __forceinline__ void dispatch_warp_run(const GemmParams& p, int32_t dispatch_warp,
                                                  uint32_t lane) {
  if (p.disp_src == nullptr) return;
  const int32_t gid = blockIdx.x * kDispatchWarps + dispatch_warp;
  const int32_t nd = gridDim.x * kDispatchWarps;
  const int32_t nb = p.disp_world * p.disp_epr;
  // buckets without rows are complete from the start
  for (int32_t q = gid * 32 + (int32_t)lane; q < nb; q += nd * 32) {
    const int32_t b = dispatch_order_bucket(q, p.disp_rank, p.disp_world, p.disp_epr);
    if (p.disp_counts[b] == 0) {
      int32_t* flag = p.disp_peer_flags[b / p.disp_epr] + p.disp_rank * p.disp_epr + (b % p.disp_epr);
      asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(p.disp_epoch) : "memory");
    }
  }
  const int32_t n_send = *p.disp_num_send;
  const int32_t chunks = p.disp_row_bytes >> 4;
  constexpr int kBatch = kDispatchSegChunks;
  const int32_t segs_per_row = (chunks + 32 * kBatch - 1) / (32 * kBatch);
  const int32_t nseg = kDispatchBatchRows * segs_per_row;
  const int32_t stride = nd * kDispatchBatchRows;
  int32_t j0 = gid * kDispatchBatchRows;
  DispatchRow row = dispatch_resolve(p, j0, n_send, nb, lane);
  while (j0 < n_send) {
    uint4 va[kBatch], vb[kBatch];
    auto seg_load = [&](int32_t sgm, uint4 (&v)[kBatch]) {
      const int32_t r = sgm / segs_per_row;
      const int32_t c0 = (sgm - r * segs_per_row) * 32 * kBatch;
      const uint8_t* src = reinterpret_cast<const uint8_t*>(
          __shfl_sync(0xffffffffu, (unsigned long long)row.src, r));
      if (src == nullptr) return;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const int32_t c = c0 + k * 32 + (int32_t)lane;
        if (c < chunks) {
          asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(v[k].x), "=r"(v[k].y), "=r"(v[k].z), "=r"(v[k].w)
                       : "l"(src + (size_t)c * 16));
        }
      }
    };
    auto seg_store = [&](int32_t sgm, const uint4 (&v)[kBatch]) {
      const int32_t r = sgm / segs_per_row;
      const int32_t c0 = (sgm - r * segs_per_row) * 32 * kBatch;
      uint8_t* dst = reinterpret_cast<uint8_t*>(
          __shfl_sync(0xffffffffu, (unsigned long long)row.dst, r));
      if (dst == nullptr) return;
#pragma unroll
      for (int k = 0; k < kBatch; ++k) {
        const int32_t c = c0 + k * 32 + (int32_t)lane;
        if (c < chunks) *reinterpret_cast<uint4*>(dst + (size_t)c * 16) = v[k];
      }
    };
    seg_load(0, va);
    for (int32_t sgm = 0; sgm < nseg; sgm += 2) {
      if (sgm + 1 < nseg) seg_load(sgm + 1, vb);
      seg_store(sgm, va);
      if (sgm + 2 < nseg) seg_load(sgm + 2, va);
      if (sgm + 1 < nseg) seg_store(sgm + 1, vb);
    }
    // the next batch's lookups overlap the draining stores of this one
    const DispatchRow next = dispatch_resolve(p, j0 + stride, n_send, nb, lane);
    // Publication of a bucket is a release chain.  Every lane orders its row stores before
    // the rows are counted at GPU scope (fence, then an acquire-release add on the counter that
    // all CTAs of this GPU share); the one thread whose add completes the bucket has thereby
    // acquired every earlier count and releases the flag at system scope.  A release is
    // cumulative, so the destination's acquire of the flag also covers the rows counted by
    // the other warps.  Only one system-scope release per bucket is issued: it drains
    // everything this GPU has in flight towards peers and the host, which is slow while host
    // copies are running.
    __threadfence();
    __syncwarp();
    if ((int32_t)lane < kDispatchBatchRows && row.bucket >= 0) {
      const int32_t b = row.bucket;
      int32_t before;
      asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;"
                   : "=r"(before)
                   : "l"(p.disp_bucket_done + b)
                   : "memory");
      if (before + 1 == p.disp_counts[b]) {
        // the last row of the bucket: leave the counter at zero for the next launch
        p.disp_bucket_done[b] = 0;
        int32_t* flag = p.disp_peer_flags[row.dst_rank] + p.disp_rank * p.disp_epr + (b % p.disp_epr);
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(p.disp_epoch)
                     : "memory");
      }
    }
    __syncwarp();
    row = next;
    j0 += stride;
  }
}

// Producer side of a fused launch: wait (bounded) until every source rank has flagged the
// rows of local expert `group` complete for this launch's epoch, then order the tensor-map
// (async proxy) reads after the flags just acquired.  False: gave up or the CTA is aborting.
__device__ __forceinline__ bool wait_expert_arrival(const GemmParams& p, int32_t group,
                                                    volatile int* abort_flag) {
  const uint64_t t0 = globaltimer_ns();
  for (int32_t src = 0; src < p.disp_world; ++src) {
    const int32_t* flag = p.disp_my_flags + src * p.disp_epr + group;
    uint32_t spins = 0;
    while (true) {
      int32_t seen;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if (seen >= p.disp_epoch) break;
      if ((++spins & 0x3f) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > kWaitBudgetNs) {
          report_status(p.status, kWaitTimeout, kSiteDispatchFlag, src * p.disp_epr + group,
                        p.disp_epoch, seen);
          *abort_flag = 1;
          return false;
        }
      }
    }
  }
  asm volatile("fence.proxy.async.global;" ::: "memory");
  return true;
}

// Order in which one CTA (or CTA pair) walks the launch's tiles.  By default every step-th
// tile.  A single-CTA ragged reduction (weight gradient) over groups with few rows can walk
// whole units instead (GemmParams::unit_walk): a unit is one (group, 256-column n-tile) and the
// CTA runs all its m-tiles back to back, so the unit's B operand stays in shared memory while
// only A streams.  Units are coarse (all m-tiles of one n-tile), so with many rows per group
// the default walk balances the SMs better and keeps the working set in L2.
struct TileCursor {
  int32_t t;       // tile index understood by decode_tile
  int32_t unit;    // unit mode: current unit
  int32_t m;       // unit mode: m-tile inside the unit
  int32_t step;
  int32_t limit;
  bool unit_mode;
  // unit mode: the unit's group, first column and reduction range, looked up once per unit
  int32_t u_group, u_n0, u_krow0, u_kcnt;
};

__device__ __forceinline__ void cursor_load_unit(TileCursor& c, const GemmParams& p) {
  if (c.unit * p.m_tiles >= c.limit) return;
  c.u_group = c.unit / p.n_tiles;
  c.u_n0 = (c.unit - c.u_group * p.n_tiles) * kBlockN;
  c.u_krow0 = p.group_offs[c.u_group];
  c.u_kcnt = p.group_offs[c.u_group + 1] - c.u_krow0;
}

// Tile under the cursor; in unit mode it comes from the cursor's cached unit, without
// divisions or table lookups.
__device__ __forceinline__ TileInfo cursor_tile(const TileCursor& c, const GemmParams& p,
                                                int32_t cta_rank) {
  if (!c.unit_mode) return decode_tile(p, c.t, cta_rank);
  TileInfo ti;
  ti.group = c.u_group;
  ti.row0 = c.m * kBlockM;
  ti.rows_valid = max(0, min(kBlockM, p.Mw - ti.row0));
  ti.n0 = c.u_n0;
  ti.krow0 = c.u_krow0;
  ti.kcnt = c.u_kcnt;
  ti.num_kb = (ti.kcnt + kBlockK - 1) / kBlockK;
  return ti;
}

template <bool kPair>
__device__ __forceinline__ TileCursor cursor_begin(const GemmParams& p, int32_t ntiles) {
  TileCursor c;
  c.unit_mode = !kPair && p.kind == kGroupedReduce && p.unit_walk != 0;
  c.limit = ntiles;
  c.m = 0;
  if (c.unit_mode) {
    c.unit = (int32_t)blockIdx.x;
    c.step = (int32_t)gridDim.x;
    c.t = c.unit * p.m_tiles;
    cursor_load_unit(c, p);
  } else {
    c.unit = 0;
    c.step = kPair ? (int32_t)(gridDim.x >> 1) : (int32_t)gridDim.x;
    c.t = kPair ? (int32_t)(blockIdx.x >> 1) : (int32_t)blockIdx.x;
  }
  return c;
}

__device__ __forceinline__ void cursor_next(TileCursor& c, const GemmParams& p) {
  if (c.unit_mode) {
    if (++c.m == p.m_tiles) {
      c.m = 0;
      c.unit += c.step;
      cursor_load_unit(c, p);
    }
    c.t = c.unit * p.m_tiles + c.m;
  } else {
    c.t += c.step;
  }
}

// Ragged reduction, last k-block of a group: rows past the group's end belong to the next
// group.  Clear them (K rows are 128 contiguous bytes in the MN-major boxes) up to the last
// 16-row MMA step that is issued; one warp, followed by a proxy fence so the tensor core sees
// the zeros.
__device__ __forceinline__ void clear_tail_rows(uint8_t* sA, uint8_t* sB, int b_boxes, bool with_b,
                                                int32_t rows_valid, int32_t ksteps, uint32_t lane) {
  const int32_t first = rows_valid * 128;
  const int32_t last = ksteps * kUmmaK * 128;
  for (int b = 0; b < 2 + b_boxes; ++b) {
    if (b >= 2 && !with_b) break;
    uint8_t* box = b < 2 ? sA + b * kBoxBytes : sB + (b - 2) * kBoxBytes;
    for (int32_t off = first + (int32_t)lane * 16; off < last; off += 32 * 16)
      *reinterpret_cast<uint4*>(box + off) = make_uint4(0, 0, 0, 0);
  }
  fence_proxy_async_smem();
  __syncwarp();
}

// kPair selects the tile mode at compile time: the single-CTA instance contains no cluster or
// cta_group::2 instruction and is launched without clusters; the pair instance needs clusters
// of two.
template <bool kPair>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint8_t* staging = smem + kStages * kStageBytes;   // == kPairStages * kPairStageBytes
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpiWarps * kStagingPerWarp);
  uint64_t* full_bar = bars;                         // [kMaxStages] this CTA's loads landed
  uint64_t* empty_bar = bars + kMaxStages;           // [kMaxStages] stage consumed by the MMA
  uint64_t* ready_bar = bars + 2 * kMaxStages;       // [kMaxStages] pair mode: both CTAs' stage ready
  uint64_t* bempty_bar = ready_bar;                  // single mode: B half of a stage consumed
  uint64_t* tmem_full = bars + 3 * kMaxStages;       // [2]
  uint64_t* tmem_empty = tmem_full + 2;              // [2]
  uint64_t* fixed_bar = tmem_empty + 2;              // [kMaxStages] single mode: tail rows cleared
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(fixed_bar + kMaxStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  constexpr bool pair = kPair;
  uint32_t cta_rank = 0;
  if constexpr (kPair) cta_rank = cluster_ctarank();
  const bool leader = cta_rank == 0;
  constexpr int nstages = kPair ? kPairStages : kStages;
  constexpr int stage_bytes = kPair ? kPairStageBytes : kStageBytes;
  // Ring geometry.  Normally a stage is [A | B] and both halves have `nstages` slots.  The
  // unit walk of a single-CTA ragged reduction keeps B resident, so only A streams and the
  // number of A bytes in flight bounds the kernel: there the memory is carved as three B slots
  // (96 KB, groups of up to 192 rows stay resident) followed by six A slots (96 KB).
  const bool compact = !kPair && p.kind == kGroupedReduce && p.unit_walk != 0;
  const int na = compact ? 6 : nstages;   // slots of the A ring (full / empty / fixed barriers)
  const int nb = compact ? 3 : nstages;   // slots of the B ring (B-consumed barriers)
  auto a_slot = [&](int i) -> uint8_t* {
    return compact ? stages + 3 * kStageBBytes + i * kStageABytes : stages + i * stage_bytes;
  };
  auto b_slot = [&](int i) -> uint8_t* {
    return compact ? stages + i * kStageBBytes : stages + i * stage_bytes + kStageABytes;
  };
  static_assert(3 * kStageBBytes + 6 * kStageABytes <= kStages * kStageBytes, "compact ring fits");
  static_assert(kMaxStages >= 6, "barrier arrays cover the compact A ring");
  constexpr int b_boxes = kPair ? 2 : 4;             // 64-column boxes of an MN-major B stage
  const int32_t b_col_off = kPair ? (int32_t)cta_rank * (kBlockN / 2) : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full_bar[s], 1);
      // single-mode ragged reduction: a stage is free once the issuing warp's MMAs have
      // consumed it and the other issuing warp and the tail warp have passed it, so none of
      // them is ever more than one phase behind the ring
      // (default walk: one issuing warp and the tail warp)
      mbar_init(&empty_bar[s],
                (!kPair && p.kind == kGroupedReduce) ? (p.unit_walk != 0 ? 3 : 2) : 1);
      // ready_bar doubles as the single-mode "B half consumed" barrier; a ragged reduction has
      // two MMA-issuing warps and both report on it
      mbar_init(&ready_bar[s], (!kPair && p.kind == kGroupedReduce) ? 2 : 1);
      mbar_init(&fixed_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], (pair ? 2 : 1) * kEpiWarps);   // one arrival per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (p.tma_store) tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    if constexpr (kPair) {
      tmem_alloc_pair(tmem_base_slot, kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_base_slot, kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync();   // the peer's barriers exist before anything arrives
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int32_t ntiles = total_tiles(p);
  // Single mode tracks the A and B halves of the stage ring separately: a ragged reduction
  // whose group fits the ring keeps B resident over the m-tiles of a unit (see TileCursor).
  // A single-CTA ragged reduction comes in two forms.  The unit walk (groups with few rows, B
  // resident over a unit's tiles) has two MMA-issuing warps and tracks the A and B rings
  // separately.  The default walk (many rows per group) uses the lean form: one lane loads,
  // one lane issues, the tail warp clears the rows past a group's end; a stage is [A | B].
  const bool lean_reduce = !kPair && p.kind == kGroupedReduce && p.unit_walk == 0;
  const bool dual_issue = !kPair && p.kind == kGroupedReduce && !lean_reduce;

  if (warp == 0 && lean_reduce) {
    // ------------------- TMA producer, ragged reduction, default walk -------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long pw_empty = 0, pw_issue = 0;
      const long long p_begin = prof_now();
      bool alive = true;
      for (int32_t t = (int32_t)blockIdx.x; t < ntiles && alive; t += (int32_t)gridDim.x) {
        const TileInfo ti = decode_tile(p, t, 0);
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          const long long c1 = prof_now();
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kSiteSmemEmpty, stage)) {
            alive = false;
            break;
          }
          const long long c8 = prof_now();
          pw_empty += c8 - c1;
          uint8_t* sA = stages + stage * kStageBytes;
          uint8_t* sB = sA + kStageABytes;
          uint64_t* fb = &full_bar[stage];
          mbar_arrive_expect_tx(fb, kStageBytes);
          const int32_t kr = ti.krow0 + kb * kBlockK;
          if (p.a_multibox) {
            tma_load_3d(sA, &tmA, fb, 0, kr, ti.row0 >> 6);
          } else {
            tma_load_2d(sA, &tmA, fb, ti.row0, kr);
            tma_load_2d(sA + kBoxBytes, &tmA, fb, ti.row0 + 64, kr);
          }
          if (p.b_multibox) {
            tma_load_4d(sB, &tmB, fb, 0, kr, ti.n0 >> 6, 0);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              tma_load_3d(sB + i * kBoxBytes, &tmB, fb, ti.n0 + 64 * i, kr, 0);
          }
          pw_issue += prof_now() - c8;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      prof_store(p, 0, pw_empty);
      prof_store(p, 1, 0);
      prof_store(p, 2, 0);
      prof_store(p, 11, pw_issue);
      prof_store(p, 12, prof_now() - p_begin);
      if (!alive) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp == 1 && lean_reduce) {
    // -------------------- MMA issuer, ragged reduction, default walk --------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t fixed_phase = 0;       // per-stage parity of the tail warp's barrier
      const uint32_t stage0 = smem_u32(stages);
      long long mw_acc = 0, mw_full = 0, mw_tail = 0, mw_issue = 0;
      const long long m_begin = prof_now();
      bool alive = true;
      for (int32_t t = (int32_t)blockIdx.x; t < ntiles && alive; t += (int32_t)gridDim.x) {
        const TileInfo ti = decode_tile(p, t, 0);
        const long long c3 = prof_now();
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kSiteTmemEmpty, acc))
          break;
        tc_fence_after_sync();
        mw_acc += prof_now() - c3;
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          const int32_t rows_left = ti.kcnt - kb * kBlockK;
          const bool tail = rows_left < kBlockK;
          const int ksteps = tail ? (rows_left + kUmmaK - 1) / kUmmaK : kBlockK / kUmmaK;
          const long long c4 = prof_now();
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kSiteSmemFull, stage)) {
            alive = false;
            break;
          }
          const long long c5 = prof_now();
          mw_full += c5 - c4;
          if (tail) {
            // the tail warp clears the rows past the group's end as soon as the block lands
            if (!mbar_wait(&fixed_bar[stage], (fixed_phase >> stage) & 1u, abort_flag, p.status,
                           kSiteSmemFull, 16 + stage)) {
              alive = false;
              break;
            }
            fixed_phase ^= 1u << stage;
            mw_tail += prof_now() - c5;
          }
          tc_fence_after_sync();
          const long long c10 = prof_now();
#ifdef MM_PROFILE
          if (p.prof_skip_mma) {
            mbar_arrive(&empty_bar[stage]);
          } else
#endif
          {
            const uint32_t a_addr = stage0 + stage * kStageBytes;
            const uint64_t a_desc = make_smem_desc(a_addr, (uint32_t)kBoxBytes, 1024);
            const uint64_t b_desc = make_smem_desc(a_addr + kStageABytes, (uint32_t)kBoxBytes, 1024);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              if (k >= ksteps) break;
              umma_f16(d_tmem, a_desc + (uint64_t)(k * (2048 >> 4)),
                       b_desc + (uint64_t)(k * (2048 >> 4)), p.idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&empty_bar[stage]);
          }
          mw_issue += prof_now() - c10;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!alive) break;
#ifdef MM_PROFILE
        if (p.prof_skip_mma) {
          mbar_arrive(&tmem_full[acc]);
        } else
#endif
        umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      prof_store(p, 3, mw_acc);
      prof_store(p, 4, mw_full);
      prof_store(p, 5, mw_tail);
      prof_store(p, 6, prof_now() - m_begin);
      prof_store(p, 13, mw_issue);
      prof_store(p, 14, 0);
    }
  } else if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      int32_t ready_group = -1;
      int bstage = 0;          // single mode: B half of the ring, advances only when B is loaded
      uint32_t bphase = 0;
      long long pw_empty = 0, pw_bempty = 0, pw_flag = 0, pw_issue = 0;
      const long long p_begin = prof_now();
      for (TileCursor cur = cursor_begin<kPair>(p, ntiles); cur.t < cur.limit && alive;
           cursor_next(cur, p)) {
        const TileInfo ti = cursor_tile(cur, p, cta_rank);
        // B stays in shared memory over the m-tiles of a unit when the group's rows fit the ring
        const bool resident = cur.unit_mode && ti.num_kb <= nb;
        const bool load_b = !resident || cur.m == 0;
        if (p.disp_src != nullptr && ti.group != ready_group) {
          const long long c0 = prof_now();
          if (!wait_expert_arrival(p, ti.group, abort_flag)) {
            alive = false;
            break;
          }
          pw_flag += prof_now() - c0;
          ready_group = ti.group;
        }
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          const long long c1 = prof_now();
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kSiteSmemEmpty, stage)) {
            alive = false;
            break;
          }
          pw_empty += prof_now() - c1;
          uint8_t* sA = a_slot(stage);
          uint8_t* sB = sA + kStageABytes;
          if constexpr (!kPair) {
            sB = b_slot(bstage);
            const long long c2 = prof_now();
            // ragged rows: A and B of a stage are consumed together, one barrier covers both
            if (p.kind == kGroupedReduce && load_b &&
                !mbar_wait(&bempty_bar[bstage], bphase ^ 1, abort_flag, p.status, kSiteSmemEmpty,
                           8 + bstage)) {
              alive = false;
              break;
            }
            pw_bempty += prof_now() - c2;
          }
          // Pair mode: both CTAs' loads count on the leader's barrier, except for the last
          // k-block of a ragged reduction whose tail rows each CTA must clear itself first;
          // that block lands on the CTA's own barrier and is handed over through ready_bar.
          const bool tail = p.kind == kGroupedReduce && ti.kcnt - kb * kBlockK < kBlockK;
          const bool direct = pair && !tail;
          if (direct) {
            if (leader) mbar_arrive_expect_tx(&full_bar[stage], 2 * stage_bytes);
          } else if (pair || load_b) {
            mbar_arrive_expect_tx(&full_bar[stage], stage_bytes);
          } else {
            mbar_arrive_expect_tx(&full_bar[stage], kStageABytes);
          }
          uint64_t* fb = &full_bar[stage];
          const long long c8 = prof_now();
          if (p.kind == kGroupedRows) {
            const int32_t k0 = kb * kBlockK;
            load2d<kPair>(direct, sA, &tmA, fb, k0, ti.row0);
            if (!p.b_mn) {
              // K-major weights: one box of 256 (or, per CTA of a pair, 128) output columns
              load3d<kPair>(direct, sB, &tmB, fb, k0, ti.n0 + b_col_off, ti.group);
            } else if (p.b_multibox == 2) {
              // fused FC1: the gate boxes and the up boxes of the tile in one instruction
              tma_load_5d(sB, &tmB, fb, 0, k0, ti.n0 >> 6, 0, ti.group);
            } else if (p.b_multibox == 1) {
              int32_t col = ti.n0 + b_col_off;
              if (p.epi == kEpiSwiglu) col = (cta_rank ? p.swiglu_F : 0) + ti.n0;   // pair: one half
              load4d<kPair>(direct, sB, &tmB, fb, 0, k0, col >> 6, ti.group);
            } else {
#pragma unroll
              for (int i = 0; i < b_boxes; ++i) {
                int32_t col;
                if (p.epi == kEpiSwiglu) {
                  // gate columns fill the first half of the 256-wide tile, up columns the second
                  const int half = pair ? (int)cta_rank : (i >> 1);
                  const int sub = pair ? i : (i & 1);
                  col = (half ? p.swiglu_F : 0) + ti.n0 + 64 * sub;
                } else {
                  col = ti.n0 + b_col_off + 64 * i;
                }
                load3d<kPair>(direct, sB + i * kBoxBytes, &tmB, fb, col, k0, ti.group);
              }
            }
          } else {
            const int32_t kr = ti.krow0 + kb * kBlockK;
            if (p.a_multibox) {
              load3d<kPair>(direct, sA, &tmA, fb, 0, kr, ti.row0 >> 6);
            } else {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                load2d<kPair>(direct, sA + i * kBoxBytes, &tmA, fb, ti.row0 + 64 * i, kr);
              }
            }
            if (load_b && p.b_multibox) {
              load4d<kPair>(direct, sB, &tmB, fb, 0, kr, (ti.n0 + b_col_off) >> 6, 0);
            } else if (load_b) {
#pragma unroll
              for (int i = 0; i < b_boxes; ++i) {
                const int32_t col = ti.n0 + b_col_off + 64 * i;
                load3d<kPair>(direct, sB + i * kBoxBytes, &tmB, fb, col, kr, 0);
              }
            }
          }
          pw_issue += prof_now() - c8;
          if (load_b && ++bstage == nb) {
            bstage = 0;
            bphase ^= 1;
          }
          if (++stage == na) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      prof_store(p, 0, pw_empty);
      prof_store(p, 1, pw_bempty);
      prof_store(p, 2, pw_flag);
      prof_store(p, 11, pw_issue);
      prof_store(p, 12, prof_now() - p_begin);
      if (!alive) {
        // Give loads already in flight time to land before the CTA retires.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else if (!kPair && warp == 1 && p.kind == kGroupedRows) {
    // ---------------------- MMA issuer, ragged rows, one CTA per tile ----------------------
    // One lane runs the whole loop: per k-block a wait for the stage, four MMAs and one commit.
    // tcgen05.mma issue blocks for about the instruction's duration, so every clock spent
    // between two issues is a clock the tensor pipe idles; the loop carries nothing else.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      const uint32_t b_lbo = p.b_mn ? (uint32_t)kBoxBytes : 16u;
      const uint64_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
      const uint32_t stage0 = smem_u32(stages);
      long long mw_acc = 0, mw_full = 0, mw_issue = 0;
      const long long m_begin = prof_now();
      bool alive = true;
      const int32_t num_kb = (p.K + kBlockK - 1) / kBlockK;
      for (int32_t t = (int32_t)blockIdx.x; t < ntiles && alive; t += (int32_t)gridDim.x) {
        const long long c3 = prof_now();
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kSiteTmemEmpty, acc))
          break;
        tc_fence_after_sync();
        mw_acc += prof_now() - c3;
        const uint32_t d_tmem = tmem_base + acc * kBlockN;
        for (int32_t kb = 0; kb < num_kb; ++kb) {
          const long long c4 = prof_now();
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kSiteSmemFull, stage)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
          const long long c5 = prof_now();
          mw_full += c5 - c4;
#ifdef MM_PROFILE
          if (p.prof_skip_mma) {
            mbar_arrive(&empty_bar[stage]);
          } else
#endif
          {
            const uint32_t a_addr = stage0 + stage * kStageBytes;
            const uint64_t a_desc = make_smem_desc(a_addr, 16u, 1024);
            const uint64_t b_desc = make_smem_desc(a_addr + kStageABytes, b_lbo, 1024);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k)
              umma_f16(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)k * b_kstep, p.idesc,
                       (kb | k) != 0 ? 1u : 0u);
            umma_commit(&empty_bar[stage]);
          }
          mw_issue += prof_now() - c5;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!alive) break;
#ifdef MM_PROFILE
        if (p.prof_skip_mma) {
          mbar_arrive(&tmem_full[acc]);
        } else
#endif
        umma_commit(&tmem_full[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
      prof_store(p, 3, mw_acc);
      prof_store(p, 4, mw_full);
      prof_store(p, 5, 0);
      prof_store(p, 6, prof_now() - m_begin);
      prof_store(p, 13, mw_issue);
      prof_store(p, 14, 0);
    }
  } else if (kPair && warp == 1 && p.kind == kGroupedRows) {
    // ---------------------- MMA issuer, ragged rows, CTA pair per tile ----------------------
    // The same lean loop on the leader CTA: both CTAs' loads complete on the leader's barrier,
    // one lane issues the cta_group::2 MMAs, and the multicast commit frees the stage in both
    // CTAs.  The peer CTA's warp has nothing to do for this problem kind.
    if constexpr (kPair) {
      if (leader && lane == 0) {
        int stage = 0;
        uint32_t phase = 0;
        int acc = 0;
        uint32_t acc_phase = 0;
        const uint32_t b_lbo = p.b_mn ? (uint32_t)kBoxBytes : 16u;
        const uint64_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
        const uint32_t stage0 = smem_u32(stages);
        bool alive = true;
        const int32_t num_kb = (p.K + kBlockK - 1) / kBlockK;
        for (int32_t t = (int32_t)(blockIdx.x >> 1); t < ntiles && alive;
             t += (int32_t)(gridDim.x >> 1)) {
          if (!mbar_wait_cluster(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status,
                                 kSiteTmemEmpty, acc))
            break;
          tc_fence_after_sync();
          const uint32_t d_tmem = tmem_base + acc * kBlockN;
          for (int32_t kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kSiteSmemFull, stage)) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
            const uint32_t a_addr = stage0 + stage * kPairStageBytes;
            const uint64_t a_desc = make_smem_desc(a_addr, 16u, 1024);
            const uint64_t b_desc = make_smem_desc(a_addr + kStageABytes, b_lbo, 1024);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k)
              umma_f16_pair(d_tmem, a_desc + (uint64_t)(k * 2), b_desc + (uint64_t)k * b_kstep,
                            p.idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit_pair(&empty_bar[stage]);
            if (++stage == kPairStages) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (!alive) break;
          umma_commit_pair(&tmem_full[acc]);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1;
        }
      }
    }
  } else if (warp == 1 || (dual_issue && warp == 3 + kEpiWarps)) {
    // ------------------------------- MMA issuer -------------------------------
    // A single-CTA ragged reduction has two issuing warps (warp 1 and the last warp): tile i of
    // this CTA's walk belongs to issuer i & 1 and accumulates in TMEM buffer i & 1, so while one
    // warp sits in its (blocking) MMA issue the other already waits for the next tile's loads,
    // tail rows and accumulator.  Both warps walk every tile and observe every stage barrier
    // in order (a parity wait cannot tell a phase from the one two phases later); each issues
    // only its own tiles.
    const int issuer = warp == 1 ? 0 : 1;
    int seq = 0;                 // tiles walked so far
    int stage = 0;
    uint32_t phase = 0;
    int acc = dual_issue ? issuer : 0;
    uint32_t acc_phase = 0;
    bool alive = true;
    uint32_t peer_full_phase = 0;   // per-stage parity of the peer CTA's own full barrier
    uint32_t ready_phase = 0;       // per-stage parity of the leader's hand-over barrier
    uint32_t fixed_phase = 0;       // per-stage parity of the tail warp's barrier (single mode)
    const uint32_t a_lbo = p.a_mn ? (uint32_t)kBoxBytes : 16u;
    const uint32_t b_lbo = p.b_mn ? (uint32_t)kBoxBytes : 16u;
    const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);
    const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
    int bstage = 0;    // single mode: next B slot of the ring
    int unit_b0 = 0;   // first B slot of the resident unit in progress
    long long mw_acc = 0, mw_full = 0, mw_tail = 0, mw_issue = 0, mw_decode = 0;
    const long long m_begin = prof_now();
    // Without pairing one lane runs the loop alone (no warp-wide step is needed, and every
    // clock between two MMA issues idles the tensor pipe); a pair needs the whole warp for the
    // tail rows and the cluster-scope waits.
    const bool run_loop = kPair || lane == 0;
    for (TileCursor cur = cursor_begin<kPair>(p, ntiles); run_loop && cur.t < cur.limit && alive;
         cursor_next(cur, p)) {
      const long long c9 = prof_now();
      const TileInfo ti = cursor_tile(cur, p, cta_rank);
      mw_decode += prof_now() - c9 + (ti.num_kb & 0);
      const bool resident = cur.unit_mode && ti.num_kb <= nb;
      const bool fresh_b = !resident || cur.m == 0;                 // B was loaded for this tile
      const bool mine = !dual_issue || (seq & 1) == issuer;
      // When B leaves shared memory.  One issuer: after the unit's last tile (or after every
      // tile when B streams).  Two issuers share a resident B, so each reports after its own
      // last tile of the unit, and the one without a tile in the unit just passes by.
      bool release_b = !resident || cur.m == p.m_tiles - 1;
      bool pass_b = false;        // not my tile, but my report on the B slots is due here
      if (dual_issue) {
        if (mine) {
          release_b = !resident || cur.m + 2 > p.m_tiles - 1;
        } else {
          release_b = false;
          pass_b = !resident || p.m_tiles == 1;
        }
      }
      if (resident && cur.m == 0) unit_b0 = bstage;
      // In pair mode only the leader CTA owns the accumulator hand-shake and issues MMAs; the
      // peer's warp still walks the stages to prepare its half of every stage.
      const long long c3 = prof_now();
      if (leader && mine) {
        bool ok = true;
        if constexpr (kPair) {
          // cluster-scope acquire: one lane polls, the warp follows
          if (lane == 0)
            ok = mbar_wait_cluster(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status,
                                   kSiteTmemEmpty, acc);
          ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        } else {
          ok = mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kSiteTmemEmpty, acc);
        }
        if (!ok) {
          alive = false;
          break;
        }
        tc_fence_after_sync();
      }
      mw_acc += prof_now() - c3;
      const uint32_t d_tmem = tmem_base + acc * kBlockN;
      for (int kb = 0; kb < ti.num_kb; ++kb) {
        const bool tail = p.kind == kGroupedReduce && ti.kcnt - kb * kBlockK < kBlockK;
        const int ksteps = tail ? (ti.kcnt - kb * kBlockK + kUmmaK - 1) / kUmmaK : kBlockK / kUmmaK;
        const bool handover = pair && tail;   // the peer prepares its half itself, then reports
        uint8_t* sA = a_slot(stage);
        uint8_t* sB = sA + kStageABytes;
        int bslot = stage;
        if constexpr (!kPair) {
          bslot = resident ? (unit_b0 + kb) % nb : bstage;
          sB = b_slot(bslot);
        }
        const long long c4 = prof_now();
        if (leader || handover) {
          // The peer's own barrier only sees the hand-over blocks, so it keeps its phases per stage.
          uint32_t par = phase;
          if (!leader) {
            par = (peer_full_phase >> stage) & 1u;
            peer_full_phase ^= 1u << stage;
          }
          if (!mbar_wait(&full_bar[stage], par, abort_flag, p.status, kSiteSmemFull, stage)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
        }
        const long long c5 = prof_now();
        mw_full += c5 - c4;
        if (tail) {
          if constexpr (kPair) {
            clear_tail_rows(sA, sB, b_boxes, fresh_b, ti.kcnt - kb * kBlockK, ksteps, lane);
          } else {
            // the tail warp clears the rows as soon as the block lands and reports here
            if (!mbar_wait(&fixed_bar[stage], (fixed_phase >> stage) & 1u, abort_flag, p.status,
                           kSiteSmemFull, 16 + stage)) {
              alive = false;
              break;
            }
            fixed_phase ^= 1u << stage;
            tc_fence_after_sync();
          }
          mw_tail += prof_now() - c5;
        }
        if constexpr (kPair) if (handover) {
          if (!leader) {
            if (lane == 0) mbar_arrive_cluster(&ready_bar[stage], 0);
          } else {
            bool ok = true;
            if (lane == 0) {
              ok = mbar_wait_cluster(&ready_bar[stage], (ready_phase >> stage) & 1u, abort_flag,
                                     p.status, kSitePairReady, stage);
            }
            ready_phase ^= 1u << stage;
            ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
            if (!ok) {
              alive = false;
              break;
            }
            tc_fence_after_sync();
          }
        }
        const long long c10 = prof_now();
        if (!mine) {
          // passing by: this warp has observed the block, the stage may be refilled once the
          // other issuer's MMAs are done
          if (lane == 0) {
            mbar_arrive(&empty_bar[stage]);
            if (pass_b) mbar_arrive(&bempty_bar[bslot]);
          }
        } else
#ifdef MM_PROFILE
        if (p.prof_skip_mma) {
          if (lane == 0) {
            mbar_arrive(&empty_bar[stage]);
            if (release_b) mbar_arrive(&bempty_bar[bslot]);
          }
        } else
#endif
        if (lane == 0 && leader) {
          const uint32_t a_addr = smem_u32(sA);
          const uint32_t b_addr = smem_u32(sB);
          const uint64_t a_desc = make_smem_desc(a_addr, a_lbo, 1024);
          const uint64_t b_desc = make_smem_desc(b_addr, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            if (k >= ksteps) break;
            if constexpr (kPair) {
              umma_f16_pair(d_tmem, a_desc + (uint64_t)(k * a_kstep),
                            b_desc + (uint64_t)(k * b_kstep), p.idesc, (kb | k) != 0 ? 1u : 0u);
            } else {
              umma_f16(d_tmem, a_desc + (uint64_t)(k * a_kstep), b_desc + (uint64_t)(k * b_kstep),
                       p.idesc, (kb | k) != 0 ? 1u : 0u);
            }
          }
          if constexpr (kPair) {
            umma_commit_pair(&empty_bar[stage]);
          } else {
            umma_commit(&empty_bar[stage]);
            if (release_b) umma_commit(&bempty_bar[bslot]);
          }
        }
        if constexpr (kPair) __syncwarp();
        mw_issue += prof_now() - c10;
        if (!resident && ++bstage == nb) bstage = 0;
        if (++stage == na) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!alive) break;
      if (resident && cur.m == p.m_tiles - 1) bstage = (unit_b0 + ti.num_kb) % nb;
      if (mine) {
#ifdef MM_PROFILE
        if (p.prof_skip_mma) {
          if (lane == 0) mbar_arrive(&tmem_full[acc]);
        } else
#endif
        if (lane == 0 && leader) {
          if constexpr (kPair) umma_commit_pair(&tmem_full[acc]); else umma_commit(&tmem_full[acc]);
        }
      }
      if constexpr (kPair) __syncwarp();
      ++seq;
      if (dual_issue) {
        if (mine) acc_phase ^= 1;        // this issuer's buffer is used once per own tile
      } else {
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
    if (lane == 0 && issuer == 0) {
      prof_store(p, 3, mw_acc);
      prof_store(p, 4, mw_full);
      prof_store(p, 5, mw_tail);
      prof_store(p, 6, prof_now() - m_begin);
      prof_store(p, 13, mw_issue);
      prof_store(p, 14, mw_decode);
    }
  } else if (warp >= 2 + kEpiWarps) {
    if (!kPair && p.kind == kGroupedReduce) {
      // --------------------------------- tail warp ---------------------------------
      // Ragged reduction in single mode: the first of the two spare warps follows the stage
      // ring and clears the rows past the group's end in each group's last k-block, off the
      // MMA warp's critical path.
      if (warp == 2 + kEpiWarps) {
        int stage = 0;
        uint32_t phase = 0;
        int bstage = 0;
        int unit_b0 = 0;
        bool alive = true;
        for (TileCursor cur = cursor_begin<kPair>(p, ntiles); cur.t < cur.limit && alive;
             cursor_next(cur, p)) {
          const TileInfo ti = cursor_tile(cur, p, cta_rank);
          const bool resident = cur.unit_mode && ti.num_kb <= nb;
          const bool fresh_b = !resident || cur.m == 0;
          if (resident && cur.m == 0) unit_b0 = bstage;
          for (int kb = 0; kb < ti.num_kb; ++kb) {
            // Wait for every block, not only the tails: the warp must never run ahead of the
            // data (a parity wait cannot tell a phase from the one two phases later).
            if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kSiteSmemFull,
                           32 + stage)) {
              alive = false;
              break;
            }
            const int32_t rows_left = ti.kcnt - kb * kBlockK;
            if (rows_left < kBlockK) {
              const int bslot = resident ? (unit_b0 + kb) % nb : bstage;
              clear_tail_rows(a_slot(stage),
                              b_slot(bslot), b_boxes, fresh_b,
                              rows_left, (rows_left + kUmmaK - 1) / kUmmaK, lane);
              if (lane == 0) mbar_arrive(&fixed_bar[stage]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (!resident && ++bstage == nb) bstage = 0;
            if (++stage == na) {
              stage = 0;
              phase ^= 1;
            }
          }
          if (resident && cur.m == p.m_tiles - 1) bstage = (unit_b0 + ti.num_kb) % nb;
        }
      }
    } else {
      // ----------------------------- dispatch warps -----------------------------
      dispatch_warp_run(p, (int32_t)(warp - 2 - kEpiWarps), lane);
    }
  } else {
    // -------------------------------- epilogue --------------------------------
    const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
    const uint32_t ew = warp - 2;
    uint8_t* stg = staging + ew * kStagingPerWarp;  // two 4 KB buffers, 1024-byte aligned
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t buf = 0;  // staging buffer the next chunk uses
    long long ew_full = 0, ew_store = 0, e_tiles = 0;
    const long long e_begin = prof_now();
    for (TileCursor cur = cursor_begin<kPair>(p, ntiles); cur.t < cur.limit; cursor_next(cur, p)) {
      const TileInfo ti = cursor_tile(cur, p, cta_rank);
      const long long c6 = prof_now();
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, kSiteTmemFull, acc)) break;
      ew_full += prof_now() - c6;
      ++e_tiles;
      tc_fence_after_sync();
      const int32_t row = q * 32 + lane;
      const int valid = row < ti.rows_valid;
      const uint32_t t_acc = tmem_base + acc * kBlockN + ((q * 32u) << 16);

      if (p.epi == kEpiSwiglu) {
        // TMEM columns 0..127 hold gate, 128..255 up, for F columns n0 .. n0 + 127.
        const int64_t grow = (int64_t)ti.row0 + row;
        uint8_t* act_ptr = reinterpret_cast<uint8_t*>(p.out + grow * p.ld_out + ti.n0);
        uint8_t* raw_ptr =
            p.out2 ? reinterpret_cast<uint8_t*>(p.out2 + grow * p.ld_out2 + ti.n0) : nullptr;
        const float w = valid ? p.row_weight[grow] : 0.0f;
        // the backward reads the received routing weights as bf16; the first column tile of
        // every row tile leaves that copy
        if (valid && ti.n0 == 0 && p.row_weight_bf16 != nullptr)
          p.row_weight_bf16[grow] = __float2bfloat16_rn(w);
        uint8_t* sa = stg;          // activation, 64 columns per pass
        uint8_t* sg = stg + 4096;   // raw gate (first half of the pass), then raw up
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            uint32_t rg[32], ru[32];
            tmem_ld_32x32(t_acc + c * 64 + h * 32, rg);
            tmem_ld_32x32(t_acc + 128 + c * 64 + h * 32, ru);
            tmem_ld_wait_regs(rg);
            tmem_ld_wait_regs(ru);
            uint32_t pa[16], pg[16], pu[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = bf16_round(__uint_as_float(rg[2 * j]));
              const float g1 = bf16_round(__uint_as_float(rg[2 * j + 1]));
              const float u0 = bf16_round(__uint_as_float(ru[2 * j]));
              const float u1 = bf16_round(__uint_as_float(ru[2 * j + 1]));
              pg[j] = pack_bf16x2(g0, g1);
              pu[j] = pack_bf16x2(u0, u1);
              pa[j] = pack_bf16x2(gated_activation(g0, u0, p) * w, gated_activation(g1, u1, p) * w);
            }
            stage_half_row(sa, lane, h * 4, pa);
            if (raw_ptr) {
              // raw rows are flushed 32 columns at a time: gate in chunks 0..3, up in 4..7
              stage_half_row(sg, lane, 0, pg);
              stage_half_row(sg, lane, 4, pu);
              __syncwarp();
              {
                const uint32_t cc = lane & 7;
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                  const uint32_t r = it * 4 + (lane >> 3);
                  const uint4 qv =
                      *reinterpret_cast<const uint4*>(sg + r * 128 + ((cc ^ (r & 7)) << 4));
                  const uint64_t pr = __shfl_sync(0xffffffffu, (unsigned long long)raw_ptr, r);
                  const int ok = __shfl_sync(0xffffffffu, valid, r);
                  if (ok) {
                    uint8_t* dst = reinterpret_cast<uint8_t*>(pr) + (c * 64 + h * 32) * 2 +
                                   (cc < 4 ? cc * 16 : (int64_t)p.swiglu_F * 2 + (cc - 4) * 16);
                    *reinterpret_cast<uint4*>(dst) = qv;
                  }
                }
              }
              __syncwarp();
            }
          }
          __syncwarp();
          flush_rows(sa, lane, act_ptr + c * 128, valid, 64);
          __syncwarp();
        }
      } else if (p.tma_store) {
        // Rectangular output tile (weight gradient): stage 32 x 64 blocks in the swizzled
        // layout and let one lane issue a tensor store per block; the map clips the edges.
        const bool zero_tile = (ti.num_kb == 0);
        const int nch = min(kBlockN / 64, (p.N - ti.n0 + 63) / 64);
        uint32_t ra[64];
        if (!zero_tile && nch > 0) tmem_ld_32x64(t_acc, ra);
#pragma unroll 1
        for (int c = 0; c < nch; ++c) {
          uint8_t* sb = stg + buf * 4096;
          // the store issued two blocks ago from this buffer must have read it
          const long long c7 = prof_now();
          if (lane == 0) bulk_wait_group_read<1>();
          __syncwarp();
          ew_store += prof_now() - c7;
          if (!zero_tile) {
            tmem_ld_wait_regs(ra);
            stage_row_f32(sb, lane, ra);
            if (c + 1 < nch) tmem_ld_32x64(t_acc + (c + 1) * 64, ra);
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              *reinterpret_cast<uint4*>(sb + lane * 128 + k * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && ti.row0 + (int32_t)q * 32 < p.Mw) {
            tma_store_3d(&tmC, sb, ti.n0 + c * 64, ti.row0 + (int32_t)q * 32, ti.group);
            bulk_commit_group();
          }
          buf ^= 1;
        }
      } else {
        uint8_t* row_ptr = nullptr;
        if (valid) {
          if (p.epi == kEpiScatter) {
            const int64_t grow = (int64_t)ti.row0 + row;
            const int32_t rk = p.row_dst_rank[grow];
            const int64_t pos = p.row_dst_pos[grow];
            row_ptr = reinterpret_cast<uint8_t*>(p.peer_bases[rk] + pos * p.ld_dst + ti.n0);
          } else if (p.kind == kGroupedRows) {
            row_ptr =
                reinterpret_cast<uint8_t*>(p.out + ((int64_t)ti.row0 + row) * p.ld_out + ti.n0);
          } else {
            row_ptr = reinterpret_cast<uint8_t*>(p.out + (int64_t)ti.group * p.out_group_stride +
                                                 ((int64_t)ti.row0 + row) * p.ld_out + ti.n0);
          }
        }
        const bool zero_tile = (ti.num_kb == 0);
        const int cols_left = p.N - ti.n0;
        const int nch = min(kBlockN / 64, (cols_left + 63) / 64);
        uint32_t ra[64];
        if (!zero_tile && nch > 0) tmem_ld_32x64(t_acc, ra);
        if (p.wide_store) {
#pragma unroll 1
          for (int c = 0; c < nch; c += 2) {
            if (!zero_tile) {
              tmem_ld_wait_regs(ra);
              stage_row_f32_wide(stg, lane, 0, ra);
              if (c + 1 < nch) {
                tmem_ld_32x64(t_acc + (c + 1) * 64, ra);
                tmem_ld_wait_regs(ra);
                stage_row_f32_wide(stg, lane, 1, ra);
              }
              if (c + 2 < nch) tmem_ld_32x64(t_acc + (c + 2) * 64, ra);
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k)
                *reinterpret_cast<uint4*>(stg + lane * 256 + k * 16) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
            flush_rows_wide(stg, lane, row_ptr + c * 128, valid, cols_left - c * 64);
            __syncwarp();
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < nch; ++c) {
            uint8_t* sb = stg + buf * 4096;
            if (!zero_tile) {
              tmem_ld_wait_regs(ra);
              stage_row_f32(sb, lane, ra);
              // the next block's TMEM load overlaps the stores of this one
              if (c + 1 < nch) tmem_ld_32x64(t_acc + (c + 1) * 64, ra);
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k)
                *reinterpret_cast<uint4*>(sb + lane * 128 + k * 16) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
            flush_rows(sb, lane, row_ptr + c * 128, valid, cols_left - c * 64);
            buf ^= 1;
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) mbar_arrive_cluster(&tmem_empty[acc], 0); else mbar_arrive(&tmem_empty[acc]);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    // every tensor store of this warp must have completed before the CTA retires
    if (p.tma_store && lane == 0) bulk_wait_group_all();
    if (ew == 0 && lane == 0) {
      prof_store(p, 7, ew_full);
      prof_store(p, 8, ew_store);
      prof_store(p, 9, prof_now() - e_begin);
      prof_store(p, 10, e_tiles);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if constexpr (kPair) cluster_sync();   // no arrival or commit may target a CTA that has left
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace mm
