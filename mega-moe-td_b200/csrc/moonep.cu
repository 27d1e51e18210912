// MoonEP load-balancing tables on the device (and the same arithmetic on the host for callers
// that hold the count matrix in host memory).
//
// Three small kernels sit between the count exchange and mm_route_finalize:
//   moonep_plan_kernel     one CTA: count cube [R, E] -> allocation, its prefix, replica slots.
//                          Every rank runs it on the same cube and gets the same plan, so the
//                          plan needs no communication.
//   moonep_cube_kernel     one CTA: plan -> balanced count cube [R, R * 2 * E/R] (every rank
//                          derives the whole cube locally, a second count exchange is not
//                          needed), plus two per-expert tables of this rank.
//   moonep_map_kernel      one thread per route: expert-major send order -> bucket-major send
//                          order over the physical slots.
// mm_route_finalize then runs unchanged on the balanced cube with 2 * E/R slots per rank.
// Around the balanced GEMMs, moonep_transport.cuh moves replica weights to the ranks that execute
// them (mm_moonep_push_replicas) and replica weight gradients back (mm_moonep_pull_replica_grads).
// Reference: src/mega_moe/kernels/moonep_planning.py:365-460 (four launches there),
// src/mega_moe/kernels/balanced_routing.py and src/mega_moe/runtime/balanced_routing.py:372-541.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "internal.h"
#include "moonep_core.h"
#include "moonep_kernels.cuh"
#include "moonep_transport.cuh"

namespace mm {
namespace {

using namespace moonep;
using namespace moonep_kernels;

int check_plan_sizes(const char* who, int stride, int world, int num_experts, int total_bin) {
  if (world <= 0 || world > kMaxWorld || num_experts <= 0 || num_experts > kMaxExperts ||
      num_experts % world != 0 || stride < num_experts ||
      (total_bin >= 0 && (total_bin < num_experts || total_bin >= stride))) {
    set_error("%s: bad sizes (world=%d experts=%d stride=%d total_bin=%d; world <= %d, "
              "experts <= %d and divisible by world)",
              who, world, num_experts, stride, total_bin, kMaxWorld, kMaxExperts);
    return MM_ERR_ARG;
  }
  return MM_OK;
}

}  // namespace
}  // namespace mm

using namespace mm;
using namespace mm::moonep;
using namespace mm::moonep_kernels;
using namespace mm::moonep_transport;

extern "C" {

int mm_moonep_plan(const int32_t* counts, int stride, int world, int num_experts, int total_bin,
                   int32_t* allocation, int32_t* alloc_cumsum, int32_t* experts_to_copy,
                   int32_t* inverse, int32_t* replica_counts, int32_t* plan_stats, void* status,
                   cudaStream_t stream) {
  if (!counts || !allocation || !alloc_cumsum || !experts_to_copy || !inverse ||
      !replica_counts || !plan_stats) {
    set_error("mm_moonep_plan: null argument");
    return MM_ERR_ARG;
  }
  if (int rc = check_plan_sizes("mm_moonep_plan", stride, world, num_experts, total_bin)) return rc;
  moonep_plan_kernel<<<1, kPlanThreads, 0, stream>>>(
      counts, stride, world, num_experts, total_bin, allocation, alloc_cumsum, experts_to_copy,
      inverse, replica_counts, plan_stats, reinterpret_cast<StatusRecord*>(status));
  return check_launch("moonep_plan_kernel");
}

int mm_moonep_plan_host(const int32_t* counts, int stride, int world, int num_experts,
                        int total_bin, int32_t* allocation, int32_t* alloc_cumsum,
                        int32_t* experts_to_copy, int32_t* inverse, int32_t* replica_counts,
                        int32_t* plan_stats) {
  if (!counts || !allocation || !alloc_cumsum || !experts_to_copy || !inverse ||
      !replica_counts || !plan_stats) {
    set_error("mm_moonep_plan_host: null argument");
    return MM_ERR_ARG;
  }
  if (int rc = check_plan_sizes("mm_moonep_plan_host", stride, world, num_experts, total_bin))
    return rc;
  const int epr = num_experts / world;
  const SerialTeam team{};
  int32_t reject = kNoReject;
  auto note = [&reject](int32_t why) { reject = why < reject ? why : reject; };
  std::vector<int32_t> transfers((size_t)world * world, 0);
  std::vector<int64_t> balance(world, 0), row_total(world, 0);
  for (int64_t i = 0; i < (int64_t)world * num_experts; ++i) {
    allocation[i] = 0;
    inverse[i] = -1;
  }
  for (int i = 0; i < world * epr; ++i) experts_to_copy[i] = -1;

  for (int e = 0; e < num_experts; ++e) {
    bool negative = false;
    int64_t total = expert_total(counts, stride, world, e, &negative);
    if (negative) note(kPlanBadCount);
    if (total > kInt32Max) {
      note(kPlanTooLarge);
      total = kInt32Max;
    }
    if (total < 0) total = 0;
    allocation[(int64_t)(e / epr) * num_experts + e] = (int32_t)total;
  }
  for (int s = 0; s < world; ++s)
    for (int e = 0; e < num_experts; ++e) row_total[s] += counts[(int64_t)s * stride + e];
  for (int h = 0; h < world; ++h)
    for (int i = 0; i < epr; ++i)
      balance[h] += allocation[(int64_t)h * num_experts + (int64_t)h * epr + i];

  const int64_t capacity = row_total[0];
  for (int s = 0; s < world; ++s) {
    if (row_total[s] != capacity) note(kPlanUnequalRows);
    if (total_bin >= 0 && counts[(int64_t)s * stride + total_bin] != row_total[s])
      note(kPlanNotDropless);
  }
  if (capacity > kInt32Max) note(kPlanTooLarge);
  if (reject == kNoReject) {
    for (int h = 0; h < world; ++h) balance[h] -= capacity;
    const int32_t rc = fill_deficits(balance.data(), transfers.data(), world);
    if (rc != kPlanOk) {
      reject = rc;
      std::fill(transfers.begin(), transfers.end(), 0);
    }
  }
  plan_stats[0] = (int32_t)(capacity > kInt32Max ? kInt32Max : (capacity < 0 ? 0 : capacity));

  for (int h = 0; h < world; ++h) {
    const int32_t rc = cut_home_group(team, h, world, epr, num_experts,
                                      transfers.data() + (size_t)h * world, allocation);
    if (rc != kPlanOk) note(rc);
  }
  int32_t most = 0;
  for (int d = 0; d < world; ++d) {
    const int32_t needed = choose_replicas(team, d, epr, num_experts, allocation,
                                           experts_to_copy, inverse);
    replica_counts[d] = needed;
    if (needed > epr) note(kPlanReplicaBudget);
    most = needed > most ? needed : most;
  }
  for (int e = 0; e < num_experts; ++e)
    allocation_prefix(allocation, world, num_experts, e, alloc_cumsum);
  plan_stats[1] = reject == kNoReject ? (int32_t)kPlanOk : reject;
  plan_stats[2] = most;
  plan_stats[3] = 0;
  return MM_OK;
}

static int check_cube_args(const char* who, const void* a, const void* b, const void* c,
                           const void* d, const void* e, const void* f, int stride, int rank,
                           int world, int num_experts, int cube_stride) {
  if (!a || !b || !c || !d || !e || !f) {
    set_error("%s: null argument", who);
    return MM_ERR_ARG;
  }
  if (int rc = check_plan_sizes(who, stride, world, num_experts, -1)) return rc;
  if (rank < 0 || rank >= world || cube_stride < 2 * num_experts) {
    set_error("%s: bad sizes (rank=%d world=%d cube_stride=%d < %d)", who, rank, world,
              cube_stride, 2 * num_experts);
    return MM_ERR_ARG;
  }
  if (a == d) {
    set_error("%s: the balanced cube must not be written over the count matrix", who);
    return MM_ERR_ARG;
  }
  return MM_OK;
}

int mm_moonep_count_cube(const int32_t* counts, int stride, int rank, int world, int num_experts,
                         const int32_t* alloc_cumsum, const int32_t* experts_to_copy,
                         int32_t* cube, int cube_stride, int32_t* expert_start, int32_t* below,
                         cudaStream_t stream) {
  if (int rc = check_cube_args("mm_moonep_count_cube", counts, alloc_cumsum, experts_to_copy,
                               cube, expert_start, below, stride, rank, world, num_experts,
                               cube_stride))
    return rc;
  moonep_cube_kernel<<<1, kCubeThreads, 0, stream>>>(counts, stride, rank, world, num_experts,
                                                     alloc_cumsum, experts_to_copy, cube,
                                                     cube_stride, expert_start, below);
  return check_launch("moonep_cube_kernel");
}

int mm_moonep_count_cube_host(const int32_t* counts, int stride, int rank, int world,
                              int num_experts, const int32_t* alloc_cumsum,
                              const int32_t* experts_to_copy, int32_t* cube, int cube_stride,
                              int32_t* expert_start, int32_t* below) {
  if (int rc = check_cube_args("mm_moonep_count_cube_host", counts, alloc_cumsum,
                               experts_to_copy, cube, expert_start, below, stride, rank, world,
                               num_experts, cube_stride))
    return rc;
  const int epr = num_experts / world;
  const int slots = 2 * epr;
  for (int b = 0; b < world * slots; ++b)
    bucket_cells(counts, stride, world, num_experts, epr, alloc_cumsum, experts_to_copy,
                 b / slots, b % slots, cube, cube_stride);
  for (int c = world * slots; c < cube_stride; ++c)
    for (int s = 0; s < world; ++s) cube[(int64_t)s * cube_stride + c] = 0;
  int32_t run = 0;
  for (int e = 0; e < num_experts; ++e) {
    below[e] = lower_rank_routes(counts, stride, rank, e);
    expert_start[e] = run;
    run += counts[(int64_t)rank * stride + e];
  }
  return MM_OK;
}

static int check_map_args(const char* who, const void* const* ptrs, int n, int num_routes,
                          int top_k, int world, int num_experts) {
  for (int i = 0; i < n; ++i) {
    if (!ptrs[i]) {
      set_error("%s: null argument", who);
      return MM_ERR_ARG;
    }
  }
  if (num_routes < 0 || top_k <= 0) {
    set_error("%s: bad sizes (num_routes=%d top_k=%d)", who, num_routes, top_k);
    return MM_ERR_ARG;
  }
  return check_plan_sizes(who, num_experts, world, num_experts, -1);
}

int mm_moonep_map_routes(const int32_t* route_in, const int32_t* expert_in,
                         const int32_t* local_stats, int num_routes, int top_k, int world,
                         int num_experts, const int32_t* expert_start, const int32_t* below,
                         const int32_t* alloc_cumsum, const int32_t* inverse,
                         const int32_t* send_bucket_starts, int32_t* send_route,
                         int32_t* send_token, int32_t* send_bucket, int32_t* route_to_send,
                         void* status, cudaStream_t stream) {
  const void* const ptrs[] = {route_in,     expert_in,  local_stats, expert_start,
                              below,        alloc_cumsum, inverse,   send_bucket_starts,
                              send_route,   send_token, send_bucket, route_to_send};
  if (int rc = check_map_args("mm_moonep_map_routes", ptrs, 12, num_routes, top_k, world,
                              num_experts))
    return rc;
  if (route_in == send_route || expert_in == send_bucket) {
    set_error("mm_moonep_map_routes: the reordered tables must not alias the inputs");
    return MM_ERR_ARG;
  }
  if (num_routes == 0) return MM_OK;
  const int blocks = (num_routes + kMapThreads - 1) / kMapThreads;
  moonep_map_kernel<<<blocks, kMapThreads, 0, stream>>>(
      route_in, expert_in, local_stats, num_routes, top_k, world, num_experts, expert_start,
      below, alloc_cumsum, inverse, send_bucket_starts, send_route, send_token, send_bucket,
      route_to_send, reinterpret_cast<StatusRecord*>(status));
  return check_launch("moonep_map_kernel");
}

int mm_moonep_map_routes_host(const int32_t* route_in, const int32_t* expert_in, int num_valid,
                              int num_routes, int top_k, int world, int num_experts,
                              const int32_t* expert_start, const int32_t* below,
                              const int32_t* alloc_cumsum, const int32_t* inverse,
                              const int32_t* send_bucket_starts, int32_t* send_route,
                              int32_t* send_token, int32_t* send_bucket, int32_t* route_to_send,
                              int32_t* num_misplaced) {
  const void* const ptrs[] = {route_in,   expert_in,  expert_start,       below,
                              alloc_cumsum, inverse,  send_bucket_starts, send_route,
                              send_token, send_bucket, route_to_send,     num_misplaced};
  if (int rc = check_map_args("mm_moonep_map_routes_host", ptrs, 12, num_routes, top_k, world,
                              num_experts))
    return rc;
  if (num_valid < 0 || num_valid > num_routes) {
    set_error("mm_moonep_map_routes_host: num_valid=%d outside [0, %d]", num_valid, num_routes);
    return MM_ERR_ARG;
  }
  int32_t bad = 0;
  for (int i = 0; i < num_valid; ++i) {
    const int32_t e = expert_in[i];
    const int32_t route = route_in[i];
    if (e < 0 || e >= num_experts || route < 0 || route >= num_routes) {
      ++bad;
      continue;
    }
    const Placement p = place_route(i, e, world, num_experts, num_experts / world, expert_start,
                                    below, alloc_cumsum, inverse, send_bucket_starts);
    if (p.bucket < 0 || p.position < 0 || p.position >= num_valid) {
      ++bad;
      continue;
    }
    send_route[p.position] = route;
    send_token[p.position] = route / top_k;
    send_bucket[p.position] = p.bucket;
    route_to_send[route] = p.position;
  }
  *num_misplaced = bad;
  return MM_OK;
}

int mm_moonep_relabel_routes(const int32_t* route_in, const int32_t* expert_in,
                             const int32_t* route_to_send, const int32_t* local_stats,
                             int num_routes, int world, int num_experts,
                             const int32_t* expert_start, const int32_t* below,
                             const int32_t* alloc_cumsum, const int32_t* inverse,
                             int32_t* physical, void* status, cudaStream_t stream) {
  const void* const ptrs[] = {route_in, expert_in,    route_to_send, local_stats, expert_start,
                              below,    alloc_cumsum, inverse,       physical};
  if (int rc = check_map_args("mm_moonep_relabel_routes", ptrs, 9, num_routes, 1, world,
                              num_experts))
    return rc;
  if (num_routes == 0) return MM_OK;
  const int blocks = (num_routes + kMapThreads - 1) / kMapThreads;
  moonep_relabel_kernel<<<blocks, kMapThreads, 0, stream>>>(
      route_in, expert_in, route_to_send, local_stats, num_routes, world, num_experts,
      expert_start, below, alloc_cumsum, inverse, physical,
      reinterpret_cast<StatusRecord*>(status));
  return check_launch("moonep_relabel_kernel");
}

static int make_transport_table(const char* who, const mm_replica_table* in, bool required,
                                TransportTable* out) {
  *out = TransportTable{nullptr, 0, 0, nullptr};
  if (!in) {
    if (!required) return MM_OK;
    set_error("%s: the first table is required", who);
    return MM_ERR_ARG;
  }
  if (!in->local || !in->peer || in->bytes <= 0 || in->bytes % 16 != 0 ||
      in->local_stride < in->bytes || in->local_stride % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(in->local) & 15) != 0) {
    set_error("%s: a table needs 16-byte aligned pointers, bytes > 0 and a multiple of 16, "
              "local_stride >= bytes and a multiple of 16 (bytes=%lld stride=%lld)",
              who, (long long)in->bytes, (long long)in->local_stride);
    return MM_ERR_ARG;
  }
  *out = TransportTable{in->local, in->local_stride, in->bytes, in->peer};
  return MM_OK;
}

static int transport_grid(const char* who, int grid_limit, int* grid) {
  if (grid_limit > 0) {
    *grid = grid_limit;
    return MM_OK;
  }
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess || sms <= 0) {
    set_error("%s: %s", who, cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  *grid = 2 * sms;
  return MM_OK;
}

static int check_transport_sizes(const char* who, const void* table, int rank, int world,
                                 int epr) {
  if (!table || world <= 0 || world > kMaxWorld || epr <= 0 || rank < 0 || rank >= world ||
      (int64_t)world * epr > kMaxListed) {
    set_error("%s: bad sizes (rank=%d world=%d experts per rank=%d; world * experts per rank "
              "<= %d)", who, rank, world, epr, kMaxListed);
    return MM_ERR_ARG;
  }
  return MM_OK;
}

int mm_moonep_push_replicas(const int32_t* experts_to_copy, int rank, int world, int epr,
                            const mm_replica_table* weights0, const mm_replica_table* weights1,
                            int grid_limit, cudaStream_t stream) {
  const char* who = "mm_moonep_push_replicas";
  if (int rc = check_transport_sizes(who, experts_to_copy, rank, world, epr)) return rc;
  TransportTable t0, t1;
  if (int rc = make_transport_table(who, weights0, true, &t0)) return rc;
  if (int rc = make_transport_table(who, weights1, false, &t1)) return rc;
  int grid = 0;
  if (int rc = transport_grid(who, grid_limit, &grid)) return rc;
  replica_push_kernel<<<grid, kTransportThreads, 0, stream>>>(experts_to_copy, rank, world, epr,
                                                              t0, t1);
  return check_launch("replica_push_kernel");
}

int mm_moonep_pull_replica_grads(const int32_t* inverse, int rank, int world, int epr,
                                 const mm_replica_table* grads0, const mm_replica_table* grads1,
                                 int grid_limit, cudaStream_t stream) {
  const char* who = "mm_moonep_pull_replica_grads";
  if (int rc = check_transport_sizes(who, inverse, rank, world, epr)) return rc;
  TransportTable t0, t1;
  if (int rc = make_transport_table(who, grads0, true, &t0)) return rc;
  if (int rc = make_transport_table(who, grads1, false, &t1)) return rc;
  int grid = 0;
  if (int rc = transport_grid(who, grid_limit, &grid)) return rc;
  replica_pull_kernel<<<grid, kTransportThreads, 0, stream>>>(inverse, rank, world, epr, t0, t1);
  return check_launch("replica_pull_kernel");
}

}  // extern "C"
