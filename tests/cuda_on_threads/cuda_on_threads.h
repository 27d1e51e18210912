// Runs CUDA kernel source on the host, one host thread per CUDA thread.  TEST INFRASTRUCTURE ONLY.
//
// Enough of the CUDA programming model for small integer kernels: __global__ / __device__ /
// __shared__, threadIdx / blockIdx, __syncthreads, __syncwarp, __shfl_xor_sync / __shfl_up_sync
// (all 32 lanes of a warp must take part, block sizes are multiples of 32), atomicMin / atomicCAS
// on int, __threadfence, uint4, __ldg, __uint_as_float / __float_as_uint, gridDim / blockDim,
// __ballot_sync, __match_any_sync, __shfl_sync, __popc, __clz, atomicAdd / atomicMax on int,
// dynamic shared memory (cot::dynamic_shared(), see the tests for how `extern __shared__` maps
// to it).
// The blocks of a launch run one after another; the threads of a block
// run concurrently as std::thread, and barriers are real barriers, so a kernel that forgets one
// can fail here as it can on a GPU.  __shared__ variables become function-local statics, which
// is what they are while one block runs at a time.  Nothing here models memory spaces, the
// memory consistency model, occupancy or timing.
#pragma once

#include <stdint.h>

#include <string.h>

#include <algorithm>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#define __CUDACC__ 1
#define __CUDA_ARCH__ 1000
#define __host__
#define __device__
#define __global__
#define __forceinline__ inline
#define __launch_bounds__(...)
#define __shared__ static

namespace cot {

class Barrier {
 public:
  explicit Barrier(int n) : n_(n) {}
  void wait() {
    std::unique_lock<std::mutex> lock(m_);
    const unsigned gen = gen_;
    if (++arrived_ == n_) {
      arrived_ = 0;
      ++gen_;
      cv_.notify_all();
    } else {
      cv_.wait(lock, [&] { return gen_ != gen; });
    }
  }

 private:
  std::mutex m_;
  std::condition_variable cv_;
  int n_;
  int arrived_ = 0;
  unsigned gen_ = 0;
};

struct Warp {
  Barrier barrier{32};
  int64_t slot[32];
};

struct Block {
  explicit Block(int threads, size_t dynamic_bytes = 0)
      : barrier(threads), warps(threads / 32), dynamic((dynamic_bytes + 15) / 16 * 16 + 16) {
    for (auto& w : warps) w = new Warp();
  }
  ~Block() {
    for (auto* w : warps) delete w;
  }
  Barrier barrier;
  std::vector<Warp*> warps;
  std::vector<unsigned char> dynamic;  // the launch's dynamic shared memory
};

struct Dim3 {
  int x, y, z;
};

struct ThreadState {
  Dim3 thread{0, 0, 0};
  Dim3 block{0, 0, 0};
  Dim3 grid{1, 1, 1};
  Dim3 block_dim{1, 1, 1};
  Block* cta = nullptr;
};

inline ThreadState& self() {
  static thread_local ThreadState s;
  return s;
}

inline Warp& my_warp() { return *self().cta->warps[self().thread.x / 32]; }

inline void* dynamic_shared() { return self().cta->dynamic.data(); }

template <class T>
T shuffle(T v, int from_lane_or_negative) {
  Warp& w = my_warp();
  const int lane = self().thread.x & 31;
  static_assert(sizeof(T) <= sizeof(int64_t), "shuffles move at most 8 bytes");
  memcpy(&w.slot[lane], &v, sizeof(T));          // the bits, not the value: T may be a float
  w.barrier.wait();
  T r = v;
  if (from_lane_or_negative >= 0) memcpy(&r, &w.slot[from_lane_or_negative], sizeof(T));
  w.barrier.wait();
  return r;
}

// body() is the kernel call; grid x block threads run it.  The host threads of a launch are
// created once and walk the blocks together (a barrier separates two blocks), which is what
// "one block at a time" means here.
template <class Body>
void launch(int grid, int block, Body body, size_t dynamic_bytes = 0) {
  Block cta(block, dynamic_bytes);
  Barrier between_blocks(block);
  std::vector<std::thread> threads;
  threads.reserve(block);
  for (int t = 0; t < block; ++t) {
    threads.emplace_back([&, t] {
      ThreadState& s = self();
      s.thread = {t, 0, 0};
      s.grid = {grid, 1, 1};
      s.block_dim = {block, 1, 1};
      s.cta = &cta;
      for (int b = 0; b < grid; ++b) {
        s.block = {b, 0, 0};
        body();
        between_blocks.wait();
      }
    });
  }
  for (auto& th : threads) th.join();
}

}  // namespace cot

#define threadIdx (::cot::self().thread)
#define blockIdx (::cot::self().block)
#define gridDim (::cot::self().grid)
#define blockDim (::cot::self().block_dim)

struct alignas(16) uint4 {
  unsigned x, y, z, w;
};

template <class T>
T __ldg(const T* p) {
  return *p;
}

inline float __uint_as_float(unsigned u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline unsigned __float_as_uint(float f) {
  unsigned u;
  memcpy(&u, &f, 4);
  return u;
}

inline void __syncthreads() { ::cot::self().cta->barrier.wait(); }
inline void __syncwarp() { ::cot::my_warp().barrier.wait(); }
inline void __threadfence() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline void __threadfence_system() { __atomic_thread_fence(__ATOMIC_SEQ_CST); }
inline void __nanosleep(unsigned) { std::this_thread::yield(); }

template <class T>
T __shfl_xor_sync(unsigned, T v, int lane_mask) {
  return ::cot::shuffle(v, (::cot::self().thread.x & 31) ^ lane_mask);
}

template <class T>
T __shfl_up_sync(unsigned, T v, int delta) {
  const int lane = ::cot::self().thread.x & 31;
  return ::cot::shuffle(v, lane >= delta ? lane - delta : -1);
}

inline unsigned __ballot_sync(unsigned, bool predicate) {
  ::cot::Warp& w = ::cot::my_warp();
  const int lane = ::cot::self().thread.x & 31;
  w.slot[lane] = predicate ? 1 : 0;
  w.barrier.wait();
  unsigned mask = 0;
  for (int i = 0; i < 32; ++i)
    if (w.slot[i]) mask |= 1u << i;
  w.barrier.wait();
  return mask;
}

template <class T>
T __shfl_sync(unsigned, T v, int src_lane) {
  return ::cot::shuffle(v, src_lane & 31);
}

inline unsigned __match_any_sync(unsigned, int value) {
  ::cot::Warp& w = ::cot::my_warp();
  const int lane = ::cot::self().thread.x & 31;
  w.slot[lane] = value;
  w.barrier.wait();
  unsigned mask = 0;
  for (int i = 0; i < 32; ++i)
    if (w.slot[i] == value) mask |= 1u << i;
  w.barrier.wait();
  return mask;
}

inline int __popc(unsigned x) { return __builtin_popcount(x); }

inline int __float_as_int(float f) {
  int i;
  memcpy(&i, &f, 4);
  return i;
}

inline int atomicAdd(int* p, int v) { return __atomic_fetch_add(p, v, __ATOMIC_SEQ_CST); }

inline int atomicMax(int* p, int v) {
  int old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  while (old < v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST,
                                                 __ATOMIC_SEQ_CST)) {
  }
  return old;
}

inline int __clz(int x) { return x == 0 ? 32 : __builtin_clz((unsigned)x); }

inline int atomicMin(int* p, int v) {
  int old = __atomic_load_n(p, __ATOMIC_SEQ_CST);
  while (old > v && !__atomic_compare_exchange_n(p, &old, v, false, __ATOMIC_SEQ_CST,
                                                 __ATOMIC_SEQ_CST)) {
  }
  return old;
}

inline int atomicCAS(int* p, int compare, int value) {
  __atomic_compare_exchange_n(p, &compare, value, false, __ATOMIC_SEQ_CST, __ATOMIC_SEQ_CST);
  return compare;
}

using std::max;
using std::min;
