// The three MoonEP kernels (see moonep.cu for what each one does and where it sits).
//
// This file uses only what it names here from its includer: mm::StatusRecord, mm::kBadIndex and
// mm::report_status (common.cuh), and the planning arithmetic of moonep_core.h.  tests/ compiles
// it a second time for the host, against a header that runs every CUDA thread as a host thread
// (barriers and warp shuffles included), to check the kernels' own text without a GPU.
#pragma once

#include "moonep_core.h"

namespace mm {
namespace moonep_kernels {

using namespace moonep;

constexpr int kPlanThreads = 256;
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kCubeThreads = 1024;
constexpr int kMapThreads = 256;
constexpr int kMaxExperts = 4096;
constexpr int32_t kPlanRejected = 4;  // mm_status_record.code
constexpr int32_t kNoReject = 0x7fffffff;

__device__ __forceinline__ int64_t warp_sum64(int64_t v) {
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
  return v;
}

__global__ void __launch_bounds__(kPlanThreads)
moonep_plan_kernel(const int32_t* __restrict__ counts, int stride, int world, int num_experts,
                   int total_bin, int32_t* __restrict__ allocation,
                   int32_t* __restrict__ alloc_cumsum, int32_t* __restrict__ experts_to_copy,
                   int32_t* __restrict__ inverse, int32_t* __restrict__ replica_counts,
                   int32_t* __restrict__ plan_stats, StatusRecord* status) {
  __shared__ int64_t row_total[kMaxWorld];
  __shared__ int64_t balance[kMaxWorld];
  __shared__ int32_t transfers[kMaxWorld * kMaxWorld];
  __shared__ int32_t reject;  // smallest PlanReject seen, kNoReject if none
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int epr = num_experts / world;
  const WarpTeam team = {lane};

  if (tid == 0) reject = kNoReject;
  for (int i = tid; i < world * world; i += kPlanThreads) transfers[i] = 0;
  for (int i = tid; i < world * num_experts; i += kPlanThreads) {
    allocation[i] = 0;
    inverse[i] = -1;
  }
  for (int i = tid; i < world * epr; i += kPlanThreads) experts_to_copy[i] = -1;
  __syncthreads();

  // B.0: routes per expert (placed on the owner's row), routes per source rank
  for (int e = tid; e < num_experts; e += kPlanThreads) {
    bool negative = false;
    int64_t total = expert_total(counts, stride, world, e, &negative);
    if (negative) atomicMin(&reject, (int32_t)kPlanBadCount);
    if (total > kInt32Max) {
      atomicMin(&reject, (int32_t)kPlanTooLarge);
      total = kInt32Max;
    }
    if (total < 0) total = 0;
    allocation[(int64_t)(e / epr) * num_experts + e] = (int32_t)total;
  }
  for (int s = warp; s < world; s += kPlanWarps) {
    int64_t mine = 0;
    for (int e = lane; e < num_experts; e += 32) mine += counts[(int64_t)s * stride + e];
    mine = warp_sum64(mine);
    if (lane == 0) row_total[s] = mine;
  }
  __syncthreads();
  for (int h = warp; h < world; h += kPlanWarps) {
    int64_t mine = 0;
    for (int i = lane; i < epr; i += 32)
      mine += allocation[(int64_t)h * num_experts + (int64_t)h * epr + i];
    mine = warp_sum64(mine);
    if (lane == 0) balance[h] = mine;
  }
  __syncthreads();

  // input checks and B.1
  if (tid == 0) {
    // only this thread touches `reject` between the two barriers around this block
    int32_t why = reject;
    const int64_t capacity = row_total[0];
    for (int s = 0; s < world; ++s) {
      if (row_total[s] != capacity) why = min(why, (int32_t)kPlanUnequalRows);
      if (total_bin >= 0 && counts[(int64_t)s * stride + total_bin] != row_total[s])
        why = min(why, (int32_t)kPlanNotDropless);
    }
    if (capacity > kInt32Max) why = min(why, (int32_t)kPlanTooLarge);
    if (why == kNoReject) {
      for (int h = 0; h < world; ++h) balance[h] -= capacity;
      const int32_t rc = fill_deficits(balance, transfers, world);
      if (rc != kPlanOk) {
        why = rc;
        for (int i = 0; i < world * world; ++i) transfers[i] = 0;
      }
    }
    reject = why;
    plan_stats[0] = (int32_t)(capacity > kInt32Max ? kInt32Max : (capacity < 0 ? 0 : capacity));
  }
  __syncthreads();

  // B.2: one warp per home rank
  for (int h = warp; h < world; h += kPlanWarps) {
    const int32_t rc = cut_home_group(team, h, world, epr, num_experts, transfers + h * world,
                                      allocation);
    if (rc != kPlanOk && lane == 0) atomicMin(&reject, rc);
  }
  __syncthreads();

  // B.3: one warp per destination rank
  for (int d = warp; d < world; d += kPlanWarps) {
    const int32_t needed = choose_replicas(team, d, epr, num_experts, allocation,
                                           experts_to_copy, inverse);
    if (lane == 0) {
      replica_counts[d] = needed;
      if (needed > epr) atomicMin(&reject, (int32_t)kPlanReplicaBudget);
    }
  }
  for (int e = tid; e < num_experts; e += kPlanThreads)
    allocation_prefix(allocation, world, num_experts, e, alloc_cumsum);
  __syncthreads();

  if (tid == 0) {
    int32_t most = 0;
    for (int d = 0; d < world; ++d) most = replica_counts[d] > most ? replica_counts[d] : most;
    const int32_t why = reject == kNoReject ? (int32_t)kPlanOk : reject;
    plan_stats[1] = why;
    plan_stats[2] = most;
    plan_stats[3] = 0;
    if (why != kPlanOk) report_status(status, kPlanRejected, why, 0, 0, 0);
  }
}

// Block-wide exclusive scan of one value per thread (kCubeThreads threads).
__device__ __forceinline__ int cube_block_scan(int v, int* warp_sums) {
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
    const int s = warp_sums[lane];
    int sinc = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, sinc, d);
      if (lane >= d) sinc += t;
    }
    warp_sums[lane] = sinc - s;
  }
  __syncthreads();
  return warp_sums[w] + inc - v;
}

__global__ void __launch_bounds__(kCubeThreads, 1)
moonep_cube_kernel(const int32_t* __restrict__ counts, int stride, int rank, int world,
                   int num_experts, const int32_t* __restrict__ alloc_cumsum,
                   const int32_t* __restrict__ experts_to_copy, int32_t* __restrict__ cube,
                   int cube_stride, int32_t* __restrict__ expert_start,
                   int32_t* __restrict__ below) {
  __shared__ int warp_sums[32];
  const int tid = threadIdx.x;
  const int epr = num_experts / world;
  const int slots = 2 * epr;
  const int buckets = world * slots;
  for (int b = tid; b < buckets; b += kCubeThreads)
    bucket_cells(counts, stride, world, num_experts, epr, alloc_cumsum, experts_to_copy,
                 b / slots, b % slots, cube, cube_stride);
  for (int c = buckets + tid; c < cube_stride; c += kCubeThreads)
    for (int s = 0; s < world; ++s) cube[(int64_t)s * cube_stride + c] = 0;
  for (int e = tid; e < num_experts; e += kCubeThreads)
    below[e] = lower_rank_routes(counts, stride, rank, e);

  // expert_start: exclusive scan of this rank's row, a run of experts per thread
  const int per = (num_experts + kCubeThreads - 1) / kCubeThreads;
  const int first = tid * per;
  const int32_t* mine = counts + (int64_t)rank * stride;
  int local = 0;
  for (int j = 0; j < per; ++j)
    if (first + j < num_experts) local += mine[first + j];
  int off = cube_block_scan(local, warp_sums);
  for (int j = 0; j < per; ++j) {
    if (first + j < num_experts) {
      expert_start[first + j] = off;
      off += mine[first + j];
    }
  }
}

__global__ void __launch_bounds__(kMapThreads)
moonep_map_kernel(const int32_t* __restrict__ route_in, const int32_t* __restrict__ expert_in,
                  const int32_t* __restrict__ local_stats, int num_routes, int top_k, int world,
                  int num_experts, const int32_t* __restrict__ expert_start,
                  const int32_t* __restrict__ below, const int32_t* __restrict__ alloc_cumsum,
                  const int32_t* __restrict__ inverse,
                  const int32_t* __restrict__ send_bucket_starts, int32_t* __restrict__ send_route,
                  int32_t* __restrict__ send_token, int32_t* __restrict__ send_bucket,
                  int32_t* __restrict__ route_to_send, StatusRecord* status) {
  const int i = blockIdx.x * kMapThreads + threadIdx.x;
  int valid = local_stats[0];
  if (valid > num_routes) valid = num_routes;
  if (i >= valid) return;
  const int32_t e = expert_in[i];
  const int32_t route = route_in[i];
  if (e < 0 || e >= num_experts || route < 0 || route >= num_routes) {
    report_status(status, kBadIndex, 0, i, e, route);
    return;
  }
  const Placement p = place_route(i, e, world, num_experts, num_experts / world, expert_start,
                                  below, alloc_cumsum, inverse, send_bucket_starts);
  if (p.bucket < 0 || p.position < 0 || p.position >= valid) {
    report_status(status, kBadIndex, 1, i, p.bucket, p.position);
    return;
  }
  send_route[p.position] = route;
  send_token[p.position] = route / top_k;
  send_bucket[p.position] = p.bucket;
  route_to_send[route] = p.position;
}

// MoonEP as a re-labelling: physical[t, j] = bucket (rank * 2 * E/R + slot) that executes route
// (t, j), -1 for a route the filter dropped.  Routing `physical` as expert ids of a layer with
// 2 * E experts reproduces the balanced send order, cube and offsets.
__global__ void __launch_bounds__(kMapThreads)
moonep_relabel_kernel(const int32_t* __restrict__ route_in, const int32_t* __restrict__ expert_in,
                      const int32_t* __restrict__ route_to_send,
                      const int32_t* __restrict__ local_stats, int num_routes, int world,
                      int num_experts, const int32_t* __restrict__ expert_start,
                      const int32_t* __restrict__ below, const int32_t* __restrict__ alloc_cumsum,
                      const int32_t* __restrict__ inverse, int32_t* __restrict__ physical,
                      StatusRecord* status) {
  const int i = blockIdx.x * kMapThreads + threadIdx.x;
  if (i >= num_routes) return;
  if (route_to_send[i] < 0) physical[i] = -1;  // flat route i was dropped
  int valid = local_stats[0];
  if (valid > num_routes) valid = num_routes;
  if (i >= valid) return;
  const int32_t e = expert_in[i];
  const int32_t route = route_in[i];
  if (e < 0 || e >= num_experts || route < 0 || route >= num_routes) {
    report_status(status, kBadIndex, 2, i, e, route);
    return;
  }
  int32_t ordinal, share_lo;
  const int32_t bucket = route_bucket(i, e, world, num_experts, num_experts / world, expert_start,
                                      below, alloc_cumsum, inverse, &ordinal, &share_lo);
  if (bucket < 0) report_status(status, kBadIndex, 3, i, e, route);
  physical[route] = bucket;
}

}  // namespace moonep_kernels
}  // namespace mm
