// MoonEP replica transport: the two byte movers around the balanced GEMMs.
//
//   replica_push_kernel   owner-push of expert weights.  Every rank scans the same
//                         experts_to_copy[destination, replica slot] table and stores the
//                         experts it owns into those slots of the destinations' replica tables
//                         (peer stores over NVLink).  Reference:
//                         src/mega_moe/kernels/replica_weight_prefetch.py:17-180.
//   replica_pull_kernel   owner-pull of weight gradients.  The balanced backward leaves one
//                         weight gradient per physical slot; the gradient in a replica slot
//                         belongs to the expert's home rank, which reads every copy (peer loads)
//                         and adds it onto its own gradient in fp32, peers in ascending order,
//                         one rounding to bf16 at the end.  Reference:
//                         src/mega_moe/kernels/replica_grad_reduce.py:62-190 (fp32 accumulation in
//                         (peer, slot) order onto the home seed).
//
// Both are persistent grids of kTransportThreads threads.  A CTA first lists its rank's work
// (owned replica slots / home experts with copies) in a fixed order in shared memory, then the
// CTAs share the list as (entry, 16 KB chunk) items, blockIdx-strided; a thread moves four
// 16-byte vectors per chunk.  No waits: the caller orders the launches with the rank barrier.
//
// Like moonep_kernels.cuh this file compiles for the host against tests/cuda_on_threads.
#pragma once

#include <stdint.h>

namespace mm {
namespace moonep_transport {

constexpr int kTransportThreads = 256;
constexpr int kVectorsPerThread = 4;
constexpr int kChunkVectors = kTransportThreads * kVectorsPerThread;  // 16 KB
constexpr int kMaxListed = 4096;                                      // world * E/R, or E/R

struct TransportTable {
  const void* local;       // push: home weights [E/R][...];  pull: home gradients (read and written)
  int64_t local_stride;    // bytes between experts of the local table
  int64_t bytes;           // bytes per expert, a multiple of 16
  void* const* peer;       // device array of `world` pointers: rank d's replica table
                           // [E/R slots][bytes], slots contiguous
};

// Exclusive scan of one value per thread over the block; returns the offset, *total the sum.
__device__ __forceinline__ int transport_block_scan(int v, int* warp_sums, int* total) {
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
    const int s = lane < kTransportThreads / 32 ? warp_sums[lane] : 0;
    int sinc = s;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, sinc, d);
      if (lane >= d) sinc += t;
    }
    if (lane < kTransportThreads / 32) warp_sums[lane] = sinc - s;
    if (lane == 31) *total = sinc;
  }
  __syncthreads();
  return warp_sums[w] + inc - v;
}

// listed[0..n): the indices i of [0, count) with keep(i), ascending; every thread gets n.
template <class Keep>
__device__ __forceinline__ int list_in_order(int count, Keep keep, int32_t* listed,
                                             int* warp_sums, int* total) {
  const int per = (count + kTransportThreads - 1) / kTransportThreads;
  const int first = threadIdx.x * per;
  int mine = 0;
  for (int j = 0; j < per; ++j)
    if (first + j < count && keep(first + j)) ++mine;
  int at = transport_block_scan(mine, warp_sums, total);
  for (int j = 0; j < per; ++j)
    if (first + j < count && keep(first + j)) listed[at++] = first + j;
  __syncthreads();
  return *total;
}

__global__ void __launch_bounds__(kTransportThreads)
replica_push_kernel(const int32_t* __restrict__ experts_to_copy, int rank, int world, int epr,
                    TransportTable t0, TransportTable t1) {
  __shared__ int32_t listed[kMaxListed];
  __shared__ int warp_sums[32];
  __shared__ int total;
  const int n = list_in_order(
      world * epr,
      [&](int i) {
        const int32_t e = experts_to_copy[i];
        return e >= 0 && e / epr == rank && i / epr != rank;
      },
      listed, warp_sums, &total);
  const int64_t vec0 = t0.bytes / 16, vec1 = t1.local ? t1.bytes / 16 : 0;
  const int64_t chunks0 = (vec0 + kChunkVectors - 1) / kChunkVectors;
  const int64_t chunks1 = (vec1 + kChunkVectors - 1) / kChunkVectors;
  const int64_t per_entry = chunks0 + chunks1;
  for (int64_t item = blockIdx.x; item < n * per_entry; item += gridDim.x) {
    const int entry = listed[item / per_entry];
    int64_t chunk = item % per_entry;
    const bool second = chunk >= chunks0;
    if (second) chunk -= chunks0;
    const TransportTable& t = second ? t1 : t0;
    const int64_t vectors = second ? vec1 : vec0;
    const int dest = entry / epr, slot = entry % epr;
    const int local_expert = experts_to_copy[entry] % epr;
    const uint4* src = reinterpret_cast<const uint4*>(
        static_cast<const char*>(t.local) + local_expert * t.local_stride);
    uint4* dst = reinterpret_cast<uint4*>(static_cast<char*>(t.peer[dest]) + slot * t.bytes);
    const int64_t base = chunk * kChunkVectors + threadIdx.x;
    uint4 v[kVectorsPerThread];
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const int64_t i = base + (int64_t)j * kTransportThreads;
      if (i < vectors) v[j] = __ldg(src + i);
    }
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const int64_t i = base + (int64_t)j * kTransportThreads;
      if (i < vectors) dst[i] = v[j];
    }
  }
}

// two bf16 values in one 32-bit word <-> two floats
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t bf16_round(float f) {  // round to nearest even, NaN stays NaN
  const uint32_t u = __float_as_uint(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x0040u;
  return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}
__device__ __forceinline__ uint32_t bf16_pack(float lo, float hi) {
  return bf16_round(lo) | (bf16_round(hi) << 16);
}

__global__ void __launch_bounds__(kTransportThreads)
replica_pull_kernel(const int32_t* __restrict__ inverse, int rank, int world, int epr,
                    TransportTable t0, TransportTable t1) {
  __shared__ int32_t listed[kMaxListed];
  __shared__ int warp_sums[32];
  __shared__ int total;
  const int num_experts = world * epr;
  // home experts of this rank that have a copy on some other rank
  const int n = list_in_order(
      epr,
      [&](int local) {
        for (int d = 0; d < world; ++d)
          if (d != rank && inverse[(int64_t)d * num_experts + rank * epr + local] >= 0) return true;
        return false;
      },
      listed, warp_sums, &total);
  const int64_t vec0 = t0.bytes / 16, vec1 = t1.local ? t1.bytes / 16 : 0;
  const int64_t chunks0 = (vec0 + kChunkVectors - 1) / kChunkVectors;
  const int64_t chunks1 = (vec1 + kChunkVectors - 1) / kChunkVectors;
  const int64_t per_entry = chunks0 + chunks1;
  for (int64_t item = blockIdx.x; item < n * per_entry; item += gridDim.x) {
    const int local = listed[item / per_entry];
    int64_t chunk = item % per_entry;
    const bool second = chunk >= chunks0;
    if (second) chunk -= chunks0;
    const TransportTable& t = second ? t1 : t0;
    const int64_t vectors = second ? vec1 : vec0;
    uint4* home = reinterpret_cast<uint4*>(
        static_cast<char*>(const_cast<void*>(t.local)) + local * t.local_stride);
    const int64_t base = chunk * kChunkVectors + threadIdx.x;
    float acc[kVectorsPerThread][8];
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const int64_t i = base + (int64_t)j * kTransportThreads;
      if (i < vectors) {
        const uint4 h = home[i];
        acc[j][0] = bf16_lo(h.x); acc[j][1] = bf16_hi(h.x);
        acc[j][2] = bf16_lo(h.y); acc[j][3] = bf16_hi(h.y);
        acc[j][4] = bf16_lo(h.z); acc[j][5] = bf16_hi(h.z);
        acc[j][6] = bf16_lo(h.w); acc[j][7] = bf16_hi(h.w);
      }
    }
    for (int d = 0; d < world; ++d) {
      if (d == rank) continue;
      const int32_t slot = inverse[(int64_t)d * num_experts + rank * epr + local];
      if (slot < 0) continue;
      const uint4* copy = reinterpret_cast<const uint4*>(
          static_cast<const char*>(t.peer[d]) + slot * t.bytes);
      uint4 r[kVectorsPerThread];
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const int64_t i = base + (int64_t)j * kTransportThreads;
        if (i < vectors) r[j] = copy[i];
      }
#pragma unroll
      for (int j = 0; j < kVectorsPerThread; ++j) {
        const int64_t i = base + (int64_t)j * kTransportThreads;
        if (i < vectors) {
          acc[j][0] += bf16_lo(r[j].x); acc[j][1] += bf16_hi(r[j].x);
          acc[j][2] += bf16_lo(r[j].y); acc[j][3] += bf16_hi(r[j].y);
          acc[j][4] += bf16_lo(r[j].z); acc[j][5] += bf16_hi(r[j].z);
          acc[j][6] += bf16_lo(r[j].w); acc[j][7] += bf16_hi(r[j].w);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < kVectorsPerThread; ++j) {
      const int64_t i = base + (int64_t)j * kTransportThreads;
      if (i < vectors) {
        uint4 h;
        h.x = bf16_pack(acc[j][0], acc[j][1]);
        h.y = bf16_pack(acc[j][2], acc[j][3]);
        h.z = bf16_pack(acc[j][4], acc[j][5]);
        h.w = bf16_pack(acc[j][6], acc[j][7]);
        home[i] = h;
      }
    }
  }
}

}  // namespace moonep_transport
}  // namespace mm
