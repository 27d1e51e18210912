// Routing metadata kernels: route filter, stable expert-major counting sort, local count
// row, and the offset tables derived from the replicated count cube.
//
// The sort is a three-pass counting sort whose result does not depend on scheduling:
//   1. every block histograms a fixed, contiguous chunk of routes;
//   2. one block turns the per-block histograms into exclusive offsets per expert and
//      scans the expert totals into bucket starts;
//   3. every block revisits its chunk in order and ranks each route among the equal
//      keys that precede it (warp match + per-warp counts), so ties keep ascending
//      route order exactly like a stable sort.
#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace mm {

constexpr int kRouteChunk = 2048;
constexpr int kRouteThreads = 256;
constexpr int kRouteWarps = kRouteThreads / 32;
constexpr int kMaxBins = 4096;

__global__ void __launch_bounds__(kRouteThreads)
route_hist_kernel(const int32_t* __restrict__ selected, int n, int num_experts, int bins,
                  int32_t* __restrict__ block_hist) {
  extern __shared__ int32_t hist[];
  for (int b = threadIdx.x; b < bins; b += kRouteThreads) hist[b] = 0;
  __syncthreads();
  const int base = blockIdx.x * kRouteChunk;
  for (int i = threadIdx.x; i < kRouteChunk; i += kRouteThreads) {
    const int r = base + i;
    if (r < n) {
      const int e = selected[r];
      if (e >= 0 && e < num_experts) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int b = threadIdx.x; b < bins; b += kRouteThreads)
    block_hist[(size_t)blockIdx.x * bins + b] = hist[b];
}

// Block-wide exclusive scan of one value per thread (1024 threads).
__device__ __forceinline__ int block_exclusive_scan_1024(int v, int* warp_sums, int* total) {
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  int inc = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, d);
    if (lane >= d) inc += t;
  }
  if (lane == 31) warp_sums[w] = inc;
  __syncthreads();
  if (w == 0) {
    int s = warp_sums[lane];
    int sinc = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, sinc, d);
      if (lane >= d) sinc += t;
    }
    warp_sums[lane] = sinc - s;
    if (lane == 31) *total = sinc;
  }
  __syncthreads();
  return warp_sums[w] + inc - v;
}

__global__ void __launch_bounds__(1024)
route_scan_kernel(int32_t* __restrict__ block_hist, int nblk, int bins,
                  int32_t* __restrict__ bucket_start, int32_t* __restrict__ count_row,
                  int32_t* __restrict__ local_stats) {
  extern __shared__ int32_t tot[];  // [bins]
  __shared__ int warp_sums[32];
  __shared__ int total;
  for (int b = threadIdx.x; b < bins; b += 1024) {
    int run = 0;
    for (int k = 0; k < nblk; ++k) {
      const size_t idx = (size_t)k * bins + b;
      const int t = block_hist[idx];
      block_hist[idx] = run;
      run += t;
    }
    tot[b] = run;
    count_row[b] = run;
  }
  __syncthreads();
  const int per = (bins + 1023) / 1024;
  const int first = threadIdx.x * per;
  int local = 0;
  for (int j = 0; j < per; ++j)
    if (first + j < bins) local += tot[first + j];
  int off = block_exclusive_scan_1024(local, warp_sums, &total);
  for (int j = 0; j < per; ++j) {
    if (first + j < bins) {
      bucket_start[first + j] = off;
      off += tot[first + j];
    }
  }
  if (threadIdx.x == 0) {
    local_stats[0] = total;
    local_stats[1] = 0;
  }
}

__global__ void __launch_bounds__(kRouteThreads)
route_scatter_kernel(const int32_t* __restrict__ selected, int n, int top_k, int num_experts,
                     int bins, const int32_t* __restrict__ block_hist,
                     const int32_t* __restrict__ bucket_start, int32_t* __restrict__ send_route,
                     int32_t* __restrict__ send_token, int32_t* __restrict__ send_bucket,
                     int32_t* __restrict__ route_to_send) {
  extern __shared__ int32_t sm[];
  int32_t* run = sm;              // [bins] next free position of each expert for this block
  int32_t* warp_cnt = sm + bins;  // [kRouteWarps][bins]
  for (int b = threadIdx.x; b < bins; b += kRouteThreads)
    run[b] = bucket_start[b] + block_hist[(size_t)blockIdx.x * bins + b];
  for (int b = threadIdx.x; b < kRouteWarps * bins; b += kRouteThreads) warp_cnt[b] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int w = threadIdx.x >> 5;
  const int base = blockIdx.x * kRouteChunk;
  for (int tile = 0; tile < kRouteChunk; tile += kRouteThreads) {
    const int r = base + tile + threadIdx.x;
    int e = -1;
    if (r < n) {
      e = selected[r];
      if (e < 0 || e >= num_experts) e = -1;
    }
    const bool valid = e >= 0;
    const unsigned mask = __match_any_sync(0xffffffffu, e);
    const int rank_w = __popc(mask & ((1u << lane) - 1u));
    const int cnt = __popc(mask);
    const bool leader = rank_w == 0;
    if (valid && leader) warp_cnt[w * bins + e] = cnt;
    __syncthreads();
    if (valid) {
      int pos = run[e] + rank_w;
      for (int w2 = 0; w2 < w; ++w2) pos += warp_cnt[w2 * bins + e];
      send_route[pos] = r;
      send_token[pos] = r / top_k;
      send_bucket[pos] = e;
      route_to_send[r] = pos;
    } else if (r < n) {
      route_to_send[r] = -1;
    }
    __syncthreads();
    if (valid && leader) {
      atomicAdd(&run[e], cnt);
      warp_cnt[w * bins + e] = 0;
    }
    __syncthreads();
  }
}

// One block.  Shared memory: tot[nb] | pre[nb] | loc[nb] | tiles[epr + 1].
__global__ void __launch_bounds__(1024)
route_finalize_kernel(const int32_t* __restrict__ cube, int rank, int world, int epr, int bins,
                      int capacity_rows, int32_t* __restrict__ send_bucket_starts,
                      int32_t* __restrict__ send_bucket_dst_starts,
                      int32_t* __restrict__ recv_counts_re, int32_t* __restrict__ recv_per_expert,
                      int32_t* __restrict__ recv_expert_offs, int32_t* __restrict__ recv_seg_starts,
                      int32_t* __restrict__ pull_dst_start, int32_t* __restrict__ stats,
                      int32_t* __restrict__ mtile_group, int32_t* __restrict__ mtile_row0,
                      int32_t* __restrict__ num_mtiles, int32_t* __restrict__ mtile2_group,
                      int32_t* __restrict__ mtile2_row0, int32_t* __restrict__ num_mtiles2,
                      int32_t* __restrict__ order_prefix, int32_t* __restrict__ bucket_done,
                      StatusRecord* status) {
  extern __shared__ int32_t sm[];
  const int nb = world * epr;
  int32_t* tot = sm;
  int32_t* pre = sm + nb;
  int32_t* loc = sm + 2 * nb;
  __shared__ int warp_sums[32];
  __shared__ int scan_total;
  __shared__ int max_required;   // largest per-destination receive total
  const int tid = threadIdx.x;
  if (tid == 0) max_required = 0;

  for (int b = tid; b < nb; b += 1024) {
    int t = 0, p = 0;
    for (int s = 0; s < world; ++s) {
      const int c = cube[(size_t)s * bins + b];
      t += c;
      if (s < rank) p += c;
    }
    tot[b] = t;
    pre[b] = p;
    loc[b] = cube[(size_t)rank * bins + b];
  }
  __syncthreads();

  // send_bucket_starts: exclusive scan of the local row over all buckets.
  {
    const int per = (nb + 1023) / 1024;
    const int first = tid * per;
    int local = 0;
    for (int j = 0; j < per; ++j)
      if (first + j < nb) local += loc[first + j];
    int off = block_exclusive_scan_1024(local, warp_sums, &scan_total);
    for (int j = 0; j < per; ++j) {
      if (first + j < nb) {
        send_bucket_starts[first + j] = off;
        off += loc[first + j];
      }
    }
  }
  __syncthreads();

  // Prefix of the local counts in dispatch order (see dispatch_order_bucket) and the
  // per-bucket delivery counters of the fused dispatch, cleared for the next launch.
  {
    const int per = (nb + 1023) / 1024;
    const int first = tid * per;
    int local = 0;
    for (int j = 0; j < per; ++j)
      if (first + j < nb) local += loc[dispatch_order_bucket(first + j, rank, world, epr)];
    int off = block_exclusive_scan_1024(local, warp_sums, &scan_total);
    for (int j = 0; j < per; ++j) {
      if (first + j < nb) {
        order_prefix[first + j] = off;
        off += loc[dispatch_order_bucket(first + j, rank, world, epr)];
      }
    }
    if (tid == 0) order_prefix[nb] = scan_total;
    for (int b = tid; b < nb; b += 1024) bucket_done[b] = 0;
  }
  __syncthreads();

  // Per destination: running base over its experts (one warp per destination, chunks of 32).
  {
    const int lane = tid & 31;
    const int w = tid >> 5;
    for (int d = w; d < world; d += 32) {
      int base = 0;
      for (int e0 = 0; e0 < epr; e0 += 32) {
        const int le = e0 + lane;
        const int b = d * epr + le;
        const int v = (le < epr) ? tot[b] : 0;
        int inc = v;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, inc, k);
          if (lane >= k) inc += t;
        }
        const int excl = base + inc - v;
        if (le < epr) {
          send_bucket_dst_starts[b] = excl + pre[b];
          if (d == rank) {
            recv_per_expert[le] = v;
            recv_expert_offs[le] = excl;
          }
        }
        base += __shfl_sync(0xffffffffu, inc, 31);
      }
      if (lane == 0) {
        stats[2 + d] = base;
        atomicMax(&max_required, base);
        if (d == rank) {
          recv_expert_offs[epr] = base;
          stats[0] = base;
        }
      }
    }
  }

  // Receive-side tables of this rank.
  for (int i = tid; i < world * epr; i += 1024) {
    const int s = i / epr;
    const int le = i - s * epr;
    recv_counts_re[i] = cube[(size_t)s * bins + rank * epr + le];
  }
  for (int le = tid; le < epr; le += 1024) {
    int run = 0;
    for (int s = 0; s < world; ++s) {
      recv_seg_starts[le * (world + 1) + s] = run;
      run += cube[(size_t)s * bins + rank * epr + le];
    }
    recv_seg_starts[le * (world + 1) + world] = run;
  }
  // pull_dst_start[le * world + s]: position of bucket (rank, le) in source s's send order.
  {
    const int lane = tid & 31;
    const int w = tid >> 5;
    const int first_bucket = rank * epr;
    for (int s = w; s < world; s += 32) {
      int base = 0;
      for (int b0 = 0; b0 < first_bucket; b0 += 32) {
        const int b = b0 + lane;
        int v = (b < first_bucket) ? cube[(size_t)s * bins + b] : 0;
#pragma unroll
        for (int k = 16; k > 0; k >>= 1) v += __shfl_xor_sync(0xffffffffu, v, k);
        base += v;
      }
      for (int e0 = 0; e0 < epr; e0 += 32) {
        const int le = e0 + lane;
        const int v = (le < epr) ? cube[(size_t)s * bins + first_bucket + le] : 0;
        int inc = v;
#pragma unroll
        for (int k = 1; k < 32; k <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, inc, k);
          if (lane >= k) inc += t;
        }
        if (le < epr) pull_dst_start[le * world + s] = base + inc - v;
        base += __shfl_sync(0xffffffffu, inc, 31);
      }
    }
  }
  __syncthreads();

  // Capacity check first: the tile tables are sized for at most capacity_rows received rows
  // (capacity / tile rows + epr entries), so on overflow no tile is written at all.
  const bool overflow = max_required > capacity_rows;
  // Row-tile tables of the local experts (128 rows per tile, and 256 for CTA pairs).
  int total_tiles[2] = {0, 0};
  for (int pass = 0; pass < 2 && !overflow; ++pass) {
    const int shift = pass == 0 ? 7 : 8;
    const int rows_per_tile = 1 << shift;
    int32_t* tg = pass == 0 ? mtile_group : mtile2_group;
    int32_t* tr = pass == 0 ? mtile_row0 : mtile2_row0;
    const int per = (epr + 1023) / 1024;
    const int first = tid * per;
    int local_tiles = 0, local_rows = 0;
    for (int j = 0; j < per; ++j) {
      if (first + j < epr) {
        const int c = tot[rank * epr + first + j];
        local_tiles += (c + rows_per_tile - 1) >> shift;
        local_rows += c;
      }
    }
    int toff = block_exclusive_scan_1024(local_tiles, warp_sums, &scan_total);
    total_tiles[pass] = scan_total;
    int roff = block_exclusive_scan_1024(local_rows, warp_sums, &scan_total);
    for (int j = 0; j < per; ++j) {
      if (first + j < epr) {
        const int c = tot[rank * epr + first + j];
        const int nt = (c + rows_per_tile - 1) >> shift;
        for (int i = 0; i < nt; ++i) {
          tg[toff + i] = first + j;
          tr[toff + i] = roff + i * rows_per_tile;
        }
        toff += nt;
        roff += c;
      }
    }
    __syncthreads();
  }
  if (tid == 0) {
    stats[1] = max_required;
    if (overflow) {
      report_status(status, kCapacityOverflow, 0, 0, capacity_rows, max_required);
      *num_mtiles = 0;
      *num_mtiles2 = 0;
    } else {
      *num_mtiles = total_tiles[0];
      *num_mtiles2 = total_tiles[1];
    }
  }
}

// Per received row: the rank that sent it and the row's position in that rank's send order.
// One warp per (local expert, source) segment.  Optionally also the permutation between this
// receive order (expert-major, then source) and the source-major "arrival" order of an
// all-to-all (source-major, then expert): row_arrival[row] = arrival index of the row,
// arrival_row = its inverse.
__global__ void __launch_bounds__(256)
route_row_tables_kernel(const int32_t* __restrict__ recv_expert_offs,
                        const int32_t* __restrict__ recv_seg_starts,
                        const int32_t* __restrict__ pull_dst_start,
                        const int32_t* __restrict__ recv_counts_re, int world, int epr,
                        int capacity_rows, int32_t* __restrict__ row_src_rank,
                        int32_t* __restrict__ row_src_pos, int32_t* __restrict__ row_arrival,
                        int32_t* __restrict__ arrival_row) {
  extern __shared__ int32_t src_start[];   // [world] rows received from the sources before s
  const bool want_perm = row_arrival != nullptr;
  if (want_perm) {
    for (int s = threadIdx.x; s < world; s += blockDim.x) {
      int t = 0;
      for (int e = 0; e < epr; ++e) t += recv_counts_re[s * epr + e];
      src_start[s] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int s = 0; s < world; ++s) {
        const int t = src_start[s];
        src_start[s] = run;
        run += t;
      }
    }
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int nseg = world * epr;
  for (int seg = blockIdx.x * warps_per_block + (threadIdx.x >> 5); seg < nseg;
       seg += gridDim.x * warps_per_block) {
    const int le = seg / world;
    const int s = seg - le * world;
    const int seg0 = recv_seg_starts[le * (world + 1) + s];
    const int cnt = recv_seg_starts[le * (world + 1) + s + 1] - seg0;
    const int row0 = recv_expert_offs[le] + seg0;
    const int pos0 = pull_dst_start[le * world + s];
    // the rows of source s arrive in its send order, which starts at this rank's expert 0
    const int arr0 = want_perm ? src_start[s] + pos0 - pull_dst_start[s] : 0;
    for (int i = lane; i < cnt; i += 32) {
      const int row = row0 + i;
      if (row < capacity_rows) {
        row_src_rank[row] = s;
        row_src_pos[row] = pos0 + i;
        if (want_perm) {
          row_arrival[row] = arr0 + i;
          if (arr0 + i < capacity_rows) arrival_row[arr0 + i] = row;
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// Router in front of the layer: top-k of the router logits and the softmax over the selected
// logits.  One warp per token; every lane keeps its share of the row in registers and the
// warp extracts the maximum k times, so the selected experts come out in the order of a
// stable descending sort of the row: ties (equal logits, -inf included, +0 and -0) go to the
// lower expert id and a NaN logit ranks above every number, like torch.sort / torch.topk.
// A row with fewer than k finite logits therefore still selects k distinct real experts; its
// weights follow the softmax's arithmetic (NaN when a NaN or only -inf logits are selected).
// ---------------------------------------------------------------------------------
constexpr int kRouterPerLane = 32;               // up to 1024 experts
constexpr int kRouterWarps = 4;
constexpr int32_t kRouterTaken = INT32_MIN;      // below the key of every logit, -inf included

// Order-preserving integer key of a logit: a < b <=> key(a) < key(b); NaN above +inf.
__device__ __forceinline__ int32_t router_key(float v) {
  if (v != v) return INT32_MAX;
  if (v == 0.0f) return 0;
  const int32_t b = __float_as_int(v);
  return b >= 0 ? b : (b ^ 0x7fffffff);
}

__global__ void __launch_bounds__(32 * kRouterWarps)
router_topk_kernel(const float* __restrict__ logits, int64_t ld, int tokens, int experts, int top_k,
                   int32_t* __restrict__ selected, float* __restrict__ weights) {
  const int lane = threadIdx.x & 31;
  const int token = blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (token >= tokens) return;
  const float* row = logits + (int64_t)token * ld;
  int32_t key[kRouterPerLane];
#pragma unroll
  for (int i = 0; i < kRouterPerLane; ++i) {
    const int e = i * 32 + lane;
    key[i] = e < experts ? router_key(row[e]) : kRouterTaken;
  }
  float my_logit = 0.0f;   // lane j keeps the j-th selected logit
  int my_expert = 0;
  float top = 0.0f;
  for (int j = 0; j < top_k; ++j) {
    int32_t best = kRouterTaken;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kRouterPerLane; ++i) {
      // strict > keeps the lowest expert id of this lane among equal keys
      if (key[i] > best) {
        best = key[i];
        best_e = i * 32 + lane;
      }
    }
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) {
      const int32_t ob = __shfl_xor_sync(0xffffffffu, best, k);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, k);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    // top_k <= experts, so a real (not yet taken) expert always remains
    const float best_v = row[best_e];
    if (j == 0) top = best_v;
    if (lane == j) {
      my_logit = best_v;
      my_expert = best_e;
    }
    if ((best_e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < kRouterPerLane; ++i)
        if (i == (best_e >> 5)) key[i] = kRouterTaken;
    }
  }
  // softmax over the selected logits (fp32, max-subtracted)
  const float ex = lane < top_k ? expf(my_logit - top) : 0.0f;
  float sum = ex;
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, k);
  if (lane < top_k) {
    selected[(int64_t)token * top_k + lane] = my_expert;
    weights[(int64_t)token * top_k + lane] = ex / sum;
  }
}

}  // namespace mm

using namespace mm;

extern "C" {

size_t mm_route_scratch_bytes(int num_routes, int bins) {
  if (num_routes < 0 || bins <= 0) return 0;
  const size_t nblk = ((size_t)num_routes + kRouteChunk - 1) / kRouteChunk;
  return (nblk + 1) * (size_t)bins * sizeof(int32_t);
}

int mm_route_local(const int32_t* selected, int num_routes, int top_k, int num_experts, int bins,
                   int32_t* send_route, int32_t* send_token, int32_t* send_bucket,
                   int32_t* route_to_send, int32_t* count_row, int32_t* local_stats, void* scratch,
                   size_t scratch_bytes, cudaStream_t stream) {
  if (!selected || !send_route || !send_token || !send_bucket || !route_to_send || !count_row ||
      !local_stats || !scratch) {
    set_error("mm_route_local: null argument");
    return MM_ERR_ARG;
  }
  if (num_routes < 0 || top_k <= 0 || num_experts <= 0 || bins < num_experts || bins > kMaxBins) {
    set_error("mm_route_local: bad sizes (routes=%d top_k=%d experts=%d bins=%d, bins <= %d)",
              num_routes, top_k, num_experts, bins, kMaxBins);
    return MM_ERR_ARG;
  }
  if (scratch_bytes < mm_route_scratch_bytes(num_routes, bins)) {
    set_error("mm_route_local: scratch too small (%zu < %zu)", scratch_bytes,
              mm_route_scratch_bytes(num_routes, bins));
    return MM_ERR_ARG;
  }
  const int nblk = (num_routes + kRouteChunk - 1) / kRouteChunk;
  int32_t* block_hist = reinterpret_cast<int32_t*>(scratch);
  int32_t* bucket_start = block_hist + (size_t)nblk * bins;
  static PerDeviceOnce scatter_attr;
  if (int rc = scatter_attr([] {
        cudaError_t e = cudaFuncSetAttribute(route_scatter_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (kRouteWarps + 1) * kMaxBins * (int)sizeof(int32_t));
        if (e != cudaSuccess) {
          set_error("cudaFuncSetAttribute(route_scatter_kernel): %s", cudaGetErrorString(e));
          return (int)MM_ERR_CUDA;
        }
        return (int)MM_OK;
      }))
    return rc;
  if (nblk > 0) {
    route_hist_kernel<<<nblk, kRouteThreads, bins * sizeof(int32_t), stream>>>(
        selected, num_routes, num_experts, bins, block_hist);
    if (int rc = check_launch("route_hist_kernel")) return rc;
  }
  route_scan_kernel<<<1, 1024, bins * sizeof(int32_t), stream>>>(block_hist, nblk, bins,
                                                                 bucket_start, count_row,
                                                                 local_stats);
  if (int rc = check_launch("route_scan_kernel")) return rc;
  if (nblk > 0) {
    route_scatter_kernel<<<nblk, kRouteThreads, (kRouteWarps + 1) * bins * sizeof(int32_t),
                           stream>>>(selected, num_routes, top_k, num_experts, bins, block_hist,
                                     bucket_start, send_route, send_token, send_bucket,
                                     route_to_send);
    if (int rc = check_launch("route_scatter_kernel")) return rc;
  }
  return MM_OK;
}

int mm_route_finalize(const int32_t* count_cube, int rank, int world, int epr, int bins,
                      int capacity_rows, int32_t* send_bucket_starts,
                      int32_t* send_bucket_dst_starts, int32_t* recv_counts_re,
                      int32_t* recv_per_expert, int32_t* recv_expert_offs,
                      int32_t* recv_seg_starts, int32_t* pull_dst_start, int32_t* stats,
                      int32_t* mtile_group, int32_t* mtile_row0, int32_t* num_mtiles,
                      int32_t* mtile2_group, int32_t* mtile2_row0, int32_t* num_mtiles2,
                      int32_t* row_src_rank, int32_t* row_src_pos, int32_t* order_prefix,
                      int32_t* bucket_done, int32_t* row_arrival, int32_t* arrival_row,
                      void* status, cudaStream_t stream) {
  if (!order_prefix || !bucket_done || !mtile2_group || !mtile2_row0 || !num_mtiles2) {
    set_error("mm_route_finalize: null argument");
    return MM_ERR_ARG;
  }
  if ((row_arrival == nullptr) != (arrival_row == nullptr)) {
    set_error("mm_route_finalize: row_arrival and arrival_row come together or not at all");
    return MM_ERR_ARG;
  }
  if (!count_cube || !send_bucket_starts || !send_bucket_dst_starts || !recv_counts_re ||
      !recv_per_expert || !recv_expert_offs || !recv_seg_starts || !pull_dst_start || !stats ||
      !mtile_group || !mtile_row0 || !num_mtiles || !row_src_rank || !row_src_pos) {
    set_error("mm_route_finalize: null argument");
    return MM_ERR_ARG;
  }
  const int nb = world * epr;
  if (world <= 0 || epr <= 0 || rank < 0 || rank >= world || bins < nb || nb > kMaxBins) {
    set_error("mm_route_finalize: bad sizes (rank=%d world=%d epr=%d bins=%d)", rank, world, epr,
              bins);
    return MM_ERR_ARG;
  }
  const size_t smem = (size_t)(3 * nb + epr + 1) * sizeof(int32_t);
  static PerDeviceOnce finalize_attr;
  if (int rc = finalize_attr([] {
        cudaError_t e = cudaFuncSetAttribute(route_finalize_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (4 * kMaxBins + 1) * (int)sizeof(int32_t));
        if (e != cudaSuccess) {
          set_error("cudaFuncSetAttribute(route_finalize_kernel): %s", cudaGetErrorString(e));
          return (int)MM_ERR_CUDA;
        }
        return (int)MM_OK;
      }))
    return rc;
  route_finalize_kernel<<<1, 1024, smem, stream>>>(
      count_cube, rank, world, epr, bins, capacity_rows, send_bucket_starts, send_bucket_dst_starts,
      recv_counts_re, recv_per_expert, recv_expert_offs, recv_seg_starts, pull_dst_start, stats,
      mtile_group, mtile_row0, num_mtiles, mtile2_group, mtile2_row0, num_mtiles2, order_prefix,
      bucket_done,
      reinterpret_cast<StatusRecord*>(status));
  if (int rc = check_launch("route_finalize_kernel")) return rc;
  const int nseg = world * epr;
  const int blocks = (nseg + 7) / 8;
  route_row_tables_kernel<<<blocks, 256, world * sizeof(int32_t), stream>>>(
      recv_expert_offs, recv_seg_starts, pull_dst_start, recv_counts_re, world, epr, capacity_rows,
      row_src_rank, row_src_pos, row_arrival, arrival_row);
  return check_launch("route_row_tables_kernel");
}

// ---------------------------------------------------------------------------------------
// mm_route_local_static: mm_route_local for callers that may not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or any allocating routine) on their
// hot path: an inference server whose memory pool was sized and frozen at start-up, code
// running under a memory budget that forbids growth after initialisation, or a plugin that
// is handed input and output buffers but owns no allocator.  mm_route_local needs a scratch
// buffer from its caller; this variant instead works in a fixed array that lives in the
// library's own device image, so the caller passes only inputs and outputs.
//
//  * The array is kRouteStaticScratchBytes (1 MiB) per GPU that loads the library, held
//    until the process exits.  Requests whose scratch need (mm_route_scratch_bytes) exceeds it
//    are rejected with MM_ERR_LIMIT; 1 MiB covers 522 240 routes at 1024 bins
//    ((blocks of 2048 routes + 1) x bins x 4 bytes).
//  * The first call on each device looks the array's device address up
//    (cudaGetSymbolAddress, with that device current) and caches it; make that first call
//    outside any stream capture.  Later calls on the device do no set-up.
//  * Nothing in the array has to start at zero: every word a call reads was written earlier
//    by the same call (the histogram pass writes all per-block counts, the scan pass all
//    bucket starts), so stale contents of a previous call are never observed.
//  * All calls on one device share the array.  Two calls whose kernels may overlap on the GPU
//    (different streams without an ordering between them) race; order them.
// ---------------------------------------------------------------------------------------
namespace {
constexpr size_t kRouteStaticScratchBytes = 1u << 20;
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_route_static_scratch[kRouteStaticScratchBytes];
void* g_route_static_ptr[kMaxDevices] = {};
std::mutex g_route_static_mutex;
}  // namespace

int mm_route_local_static(const int32_t* selected, int num_routes, int top_k, int num_experts,
                          int bins, int32_t* send_route, int32_t* send_token,
                          int32_t* send_bucket, int32_t* route_to_send, int32_t* count_row,
                          int32_t* local_stats, cudaStream_t stream) {
  if (num_routes < 0 || bins <= 0) {
    set_error("mm_route_local_static: bad sizes (routes=%d bins=%d)", num_routes, bins);
    return MM_ERR_ARG;
  }
  const size_t need = mm_route_scratch_bytes(num_routes, bins);
  if (need > kRouteStaticScratchBytes) {
    set_error("mm_route_local_static: %d routes at %d bins need %zu bytes of scratch, the built-in "
              "array holds %zu; use mm_route_local with caller-provided scratch",
              num_routes, bins, need, kRouteStaticScratchBytes);
    return MM_ERR_LIMIT;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    set_error("mm_route_local_static: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return MM_ERR_CUDA;
  }
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_route_static_mutex);
    if (g_route_static_ptr[dev] == nullptr) {
      // The array's name is only a host-side handle: kernels need its device address.
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_route_static_scratch);
      if (e != cudaSuccess || p == nullptr) {
        set_error("mm_route_local_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        return MM_ERR_CUDA;
      }
      g_route_static_ptr[dev] = p;
    }
    scratch = g_route_static_ptr[dev];
  }
  return mm_route_local(selected, num_routes, top_k, num_experts, bins, send_route, send_token,
                        send_bucket, route_to_send, count_row, local_stats, scratch,
                        kRouteStaticScratchBytes, stream);
}

int mm_router_topk(const float* logits, int64_t ld_logits, int tokens, int num_experts, int top_k,
                   int32_t* selected, float* weights, cudaStream_t stream) {
  if (!logits || !selected || !weights) {
    set_error("mm_router_topk: null argument");
    return MM_ERR_ARG;
  }
  if (tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > 32 || top_k > num_experts ||
      ld_logits < num_experts) {
    set_error("mm_router_topk: need 1 <= top_k <= min(32, experts) and ld >= experts "
              "(tokens=%d experts=%d top_k=%d)", tokens, num_experts, top_k);
    return MM_ERR_ARG;
  }
  if (num_experts > 32 * kRouterPerLane) {
    set_error("mm_router_topk: %d experts exceed the limit of %d", num_experts, 32 * kRouterPerLane);
    return MM_ERR_LIMIT;
  }
  if (tokens == 0) return MM_OK;
  const int blocks = (tokens + kRouterWarps - 1) / kRouterWarps;
  router_topk_kernel<<<blocks, 32 * kRouterWarps, 0, stream>>>(logits, ld_logits, tokens, num_experts,
                                                               top_k, selected, weights);
  return check_launch("router_topk_kernel");
}

}  // extern "C"
