// The MoonEP kernels of the package (csrc/moonep_kernels.cuh, unmodified) compiled for the host
// with cuda_on_threads.h and launched with the grids of csrc/moonep.cu.  TEST INFRASTRUCTURE ONLY.
#include "cuda_on_threads.h"

namespace mm {

// what moonep_kernels.cuh takes from common.cuh on the device
struct StatusRecord {
  int32_t code, site, slot, want, seen, block, pad[2];
};
enum StatusCode : int32_t { kOk = 0, kWaitTimeout = 1, kCapacityOverflow = 2, kBadIndex = 3 };

inline void report_status(StatusRecord* st, int32_t code, int32_t site, int32_t slot,
                          int32_t want, int32_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site;
    st->slot = slot;
    st->want = want;
    st->seen = seen;
    st->block = (int32_t)blockIdx.x;
    __threadfence();
  }
}

}  // namespace mm

#include "moonep_kernels.cuh"
#include "moonep_transport.cuh"

using namespace mm;
using namespace mm::moonep_kernels;
using namespace mm::moonep_transport;

extern "C" {

void cot_moonep_plan(const int32_t* counts, int stride, int world, int num_experts, int total_bin,
                     int32_t* allocation, int32_t* alloc_cumsum, int32_t* experts_to_copy,
                     int32_t* inverse, int32_t* replica_counts, int32_t* plan_stats,
                     void* status) {
  cot::launch(1, kPlanThreads, [=] {
    moonep_plan_kernel(counts, stride, world, num_experts, total_bin, allocation, alloc_cumsum,
                       experts_to_copy, inverse, replica_counts, plan_stats,
                       static_cast<StatusRecord*>(status));
  });
}

void cot_moonep_count_cube(const int32_t* counts, int stride, int rank, int world,
                           int num_experts, const int32_t* alloc_cumsum,
                           const int32_t* experts_to_copy, int32_t* cube, int cube_stride,
                           int32_t* expert_start, int32_t* below) {
  cot::launch(1, kCubeThreads, [=] {
    moonep_cube_kernel(counts, stride, rank, world, num_experts, alloc_cumsum, experts_to_copy,
                       cube, cube_stride, expert_start, below);
  });
}

void cot_moonep_map_routes(const int32_t* route_in, const int32_t* expert_in,
                           const int32_t* local_stats, int num_routes, int top_k, int world,
                           int num_experts, const int32_t* expert_start, const int32_t* below,
                           const int32_t* alloc_cumsum, const int32_t* inverse,
                           const int32_t* send_bucket_starts, int32_t* send_route,
                           int32_t* send_token, int32_t* send_bucket, int32_t* route_to_send,
                           void* status) {
  if (num_routes == 0) return;
  const int blocks = (num_routes + kMapThreads - 1) / kMapThreads;
  cot::launch(blocks, kMapThreads, [=] {
    moonep_map_kernel(route_in, expert_in, local_stats, num_routes, top_k, world, num_experts,
                      expert_start, below, alloc_cumsum, inverse, send_bucket_starts, send_route,
                      send_token, send_bucket, route_to_send, static_cast<StatusRecord*>(status));
  });
}

void cot_moonep_relabel_routes(const int32_t* route_in, const int32_t* expert_in,
                               const int32_t* route_to_send, const int32_t* local_stats,
                               int num_routes, int world, int num_experts,
                               const int32_t* expert_start, const int32_t* below,
                               const int32_t* alloc_cumsum, const int32_t* inverse,
                               int32_t* physical, void* status) {
  if (num_routes == 0) return;
  const int blocks = (num_routes + kMapThreads - 1) / kMapThreads;
  cot::launch(blocks, kMapThreads, [=] {
    moonep_relabel_kernel(route_in, expert_in, route_to_send, local_stats, num_routes, world,
                          num_experts, expert_start, below, alloc_cumsum, inverse, physical,
                          static_cast<StatusRecord*>(status));
  });
}

// tables: local pointer, bytes between local experts, bytes per expert, array of `world` pointers
void cot_moonep_push_replicas(const int32_t* experts_to_copy, int rank, int world, int epr,
                              const void* local0, int64_t stride0, int64_t bytes0,
                              void* const* peer0, const void* local1, int64_t stride1,
                              int64_t bytes1, void* const* peer1, int grid) {
  const TransportTable t0 = {local0, stride0, bytes0, peer0};
  const TransportTable t1 = {local1, stride1, bytes1, peer1};
  cot::launch(grid, kTransportThreads,
              [=] { replica_push_kernel(experts_to_copy, rank, world, epr, t0, t1); });
}

void cot_moonep_pull_replica_grads(const int32_t* inverse, int rank, int world, int epr,
                                   void* local0, int64_t stride0, int64_t bytes0,
                                   void* const* peer0, void* local1, int64_t stride1,
                                   int64_t bytes1, void* const* peer1, int grid) {
  const TransportTable t0 = {local0, stride0, bytes0, peer0};
  const TransportTable t1 = {local1, stride1, bytes1, peer1};
  cot::launch(grid, kTransportThreads,
              [=] { replica_pull_kernel(inverse, rank, world, epr, t0, t1); });
}

}  // extern "C"
