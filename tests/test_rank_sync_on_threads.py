"""The two cross-rank synchronisation kernels of mega-moe-td_b200/csrc/movement.cu on the host,
all ranks concurrently: ``count_exchange_kernel`` (count rows by peer stores behind an epoch flag,
two cubes used alternately) and ``rank_barrier_kernel`` (signal / wait phases).  The kernels are
cut out of the file, their release stores and acquire loads mapped onto host atomics of the same
ordering (cuda_on_threads/host_build.py::map_ptx).

Every rank runs a sequence of steps with random pauses: exchange, read its cube like the offset
kernel would, optionally signal and wait on the rank barrier.  A rank must always read exactly
the rows of its own step, however far the other ranks have run ahead; with one cube instead of
two the same schedule is caught reading a later step's rows, which is what the double buffer is
for.  A rank that never arrives ends the waits with a status record."""

from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np
import pytest

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "mega-moe-td_b200" / "csrc"
sys.path.insert(0, str(HERE))

from cuda_on_threads.host_build import compile_for_host, cut, map_ptx  # noqa: E402

HARNESS = r"""
#include <time.h>
#include <string.h>
#include <random>
#include <thread>
#include <vector>
#include "cuda_on_threads.h"

namespace mm {
struct StatusRecord {
  int32_t code, site, slot, want, seen, block, pad[2];
};
enum StatusCode : int32_t { kOk = 0, kWaitTimeout = 1 };
enum WaitSite : int32_t { kSiteRankBarrier = 5, kSiteCountFlag = 9 };
static uint64_t kWaitBudgetNs = 20000000000ull;
inline uint64_t globaltimer_ns() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
}
inline void report_status(StatusRecord* st, int32_t code, int32_t site, int32_t slot,
                          int32_t want, int32_t seen) {
  if (st == nullptr) return;
  if (atomicCAS(&st->code, 0, code) == 0) {
    st->site = site; st->slot = slot; st->want = want; st->seen = seen;
    st->block = (int32_t)blockIdx.x;
  }
}
%(barrier)s
%(exchange)s
}  // namespace mm
using namespace mm;

extern "C" void set_wait_budget_ns(uint64_t ns) { mm::kWaitBudgetNs = ns; }

// rows: [steps][world][bins]; cubes[r]: two cubes of [world][bins]; returns per rank the number
// of steps in which the cube it read differed from the rows of that step.
extern "C" void run_steps(int world, int bins, int steps, int two_cubes, int with_barrier,
                          int absent_rank, int32_t* const* cubes, int32_t* const* count_flags,
                          int32_t* const* barrier_flags, const int32_t* rows, int32_t* wrong,
                          StatusRecord* status, unsigned seed) {
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r) {
    if (r == absent_rank) continue;
    ranks.emplace_back([=] {
      std::mt19937 rng(seed + 977u * (unsigned)r);
      auto pause = [&](int scale) {
        timespec ts = {0, (long)(rng() %% (200000u * (unsigned)scale + 1u))};
        nanosleep(&ts, nullptr);
      };
      std::vector<int32_t> seen((size_t)world * bins);
      for (int step = 1; step <= steps; ++step) {
        const int32_t* mine = rows + ((size_t)(step - 1) * world + r) * bins;
        const int64_t off = two_cubes ? (int64_t)(step & 1) * world * bins : 0;
        cot::launch(1, 128, [=] {
          count_exchange_kernel(mine, bins, r, world, cubes, off, count_flags, count_flags[r], step,
                                status + r);
        });
        pause(r == 0 ? 8 : 1);                       // rank 0 is slow to read its cube
        memcpy(seen.data(), cubes[r] + off, seen.size() * sizeof(int32_t));
        pause(1);
        if (memcmp(seen.data(), rows + (size_t)(step - 1) * world * bins,
                   seen.size() * sizeof(int32_t)) != 0)
          __atomic_fetch_add(&wrong[r], 1, __ATOMIC_SEQ_CST);
        if (with_barrier) {
          cot::launch(1, 64, [=] { rank_barrier_kernel(barrier_flags, r, world, step, 1, status + r); });
          pause(2);
          cot::launch(1, 64, [=] { rank_barrier_kernel(barrier_flags, r, world, step, 2, status + r); });
        }
      }
    });
  }
  for (auto& t : ranks) t.join();
}
"""


@pytest.fixture(scope="module")
def sync(tmp_path_factory):
    movement = (CSRC / "movement.cu").read_text()
    src = HARNESS % dict(
        barrier=map_ptx(cut(movement, "__global__ void rank_barrier_kernel(")),
        exchange=map_ptx(cut(movement, "__global__ void __launch_bounds__(1024)\ncount_exchange_kernel(")),
    )
    d = tmp_path_factory.mktemp("rank_sync")
    (d / "rank_sync.cpp").write_text(src)
    lib = C.CDLL(str(compile_for_host(d / "rank_sync.cpp", d / "libranksync.so")))
    lib.run_steps.restype = None
    lib.set_wait_budget_ns.restype = None
    lib.set_wait_budget_ns.argtypes = [C.c_uint64]
    return lib


def run(sync, world, bins, steps, two_cubes=True, with_barrier=False, absent=-1, seed=1):
    rng = np.random.default_rng(seed)
    rows = rng.integers(0, 1 << 20, size=(steps, world, bins)).astype(np.int32)
    cubes = [np.full(2 * world * bins, -1, np.int32) for _ in range(world)]
    cflags = [np.zeros(world, np.int32) for _ in range(world)]
    bflags = [np.zeros(world, np.int32) for _ in range(world)]
    table = lambda arrays: (C.c_void_p * world)(*[a.ctypes.data for a in arrays])  # noqa: E731
    wrong = np.zeros(world, np.int32)
    status = np.zeros((world, 8), np.int32)
    sync.run_steps(world, bins, steps, int(two_cubes), int(with_barrier), absent, table(cubes),
                   table(cflags), table(bflags), C.c_void_p(rows.ctypes.data),
                   C.c_void_p(wrong.ctypes.data), C.c_void_p(status.ctypes.data), seed)
    return wrong, status, cflags, bflags


@pytest.mark.parametrize("world, bins", [(2, 8), (4, 64), (8, 1024)])
@pytest.mark.parametrize("with_barrier", [False, True])
def test_every_rank_reads_the_rows_of_its_own_step(sync, world, bins, with_barrier):
    steps = 12
    for seed in (1, 2, 3):
        wrong, status, cflags, bflags = run(sync, world, bins, steps, with_barrier=with_barrier,
                                            seed=seed)
        assert wrong.tolist() == [0] * world and (status[:, 0] == 0).all()
        assert all((f == steps).all() for f in cflags)
        if with_barrier:
            assert all((f == steps).all() for f in bflags)


def test_one_cube_instead_of_two_is_caught(sync):
    """The same schedule with a single cube lets a fast rank's next row land in the cube a slow
    rank is still reading; the check above must see that."""
    total = 0
    for seed in range(1, 9):
        wrong, status, _, _ = run(sync, 4, 256, 12, two_cubes=False, seed=seed)
        assert (status[:, 0] == 0).all()
        total += int(wrong.sum())
    assert total > 0


def test_an_absent_rank_ends_the_waits_with_a_status_record(sync):
    sync.set_wait_budget_ns(200_000_000)
    try:
        wrong, status, _, _ = run(sync, 3, 8, 1, with_barrier=True, absent=2)
    finally:
        sync.set_wait_budget_ns(20_000_000_000)
    for r in (0, 1):
        # code 1 (wait timed out), site 9 (count flag), slot = the absent source, wanted epoch 1
        assert status[r, :5].tolist() == [1, 9, 2, 1, 0]
