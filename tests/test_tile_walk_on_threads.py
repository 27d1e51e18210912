"""The tile walk of the persistent grouped GEMM, executed on the host from its own source text.

``GemmParams``, ``total_tiles``, ``decode_tile`` and the ``TileCursor`` functions are cut out of
mega-moe-td_b200/csrc/gemm_sm100.cuh (``TileInfo`` out of csrc/common.cuh), compiled by g++
against tests/cuda_on_threads/cuda_on_threads.h, and every CTA of a grid walks its tiles with
the loop the kernel's roles use.  For the three launch forms (ragged rows with one CTA per tile,
ragged rows with CTA pairs, ragged reduction with the default and with the unit walk) the union
of all CTAs' tiles must be exactly the set of output tiles, each once, with the row / column /
reduction ranges the tile tables imply.  The GPU suite shows this through values on the shapes
it runs; here the walk itself is checked over random groups (empty groups, one row, thousands of
rows), column counts and grid sizes."""

from __future__ import annotations

import ctypes as C
import re
import sys
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent
HERE = Path(__file__).resolve().parent
CSRC = REPO / "mega-moe-td_b200" / "csrc"
sys.path.insert(0, str(HERE))

HARNESS = r"""
#include "cuda_on_threads.h"
struct __nv_bfloat16;
namespace mm {
struct StatusRecord;
%(tile_info)s
%(constants)s
%(params)s
%(total_tiles)s
%(decode_tile)s
%(cursor)s
%(skinny)s
}  // namespace mm
using namespace mm;

// the transposed ("skinny") kernel: every role walks `for (t = blockIdx.x; t < ntiles; t += gridDim.x)`
extern "C" void walk_skinny(int epi, int swiglu_F, int n_tiles, const int32_t* group_offs,
                            const int32_t* mtile_group, const int32_t* mtile_row0,
                            const int32_t* num_mtiles, int grid, int32_t* out, int32_t* count,
                            int capacity) {
  GemmParams p = {};
  p.epi = epi; p.swiglu_F = swiglu_F; p.n_tiles = n_tiles; p.pair = 2;
  p.group_offs = group_offs; p.mtile_group = mtile_group; p.mtile_row0 = mtile_row0;
  p.num_mtiles = num_mtiles;
  cot::launch(grid, 32, [=] {
    if (threadIdx.x != 0) return;
    const int32_t ntiles = (*p.num_mtiles) * p.n_tiles;
    for (int32_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const SkinnyTile ti = skinny_tile(p, t);
      const int at = __atomic_fetch_add(count, 1, __ATOMIC_SEQ_CST);
      if (at >= capacity) continue;
      int32_t* row = out + (size_t)at * 8;
      row[0] = (int32_t)blockIdx.x; row[1] = ti.group; row[2] = ti.row0; row[3] = ti.rows_valid;
      row[4] = ti.n0; row[5] = ti.ntok; row[6] = skinny_half_col(p, ti, 0);
      row[7] = skinny_half_col(p, ti, 1);
    }
  });
}

// One host thread per CTA walks the launch like a role of the kernel does and records its tiles
// as rows of 8 ints: cta, group, row0, rows_valid, n0, num_kb, krow0, kcnt.
template <bool kPair>
static void walk(const GemmParams p, int grid, int32_t* out, int32_t* count, int capacity) {
  cot::launch(grid, 32, [=] {
    if (threadIdx.x != 0) return;
    const int32_t cta_rank = kPair ? (int32_t)(blockIdx.x & 1) : 0;
    const int32_t ntiles = total_tiles(p);
    for (TileCursor cur = cursor_begin<kPair>(p, ntiles); cur.t < cur.limit; cursor_next(cur, p)) {
      const TileInfo ti = cursor_tile(cur, p, cta_rank);
      const int at = __atomic_fetch_add(count, 1, __ATOMIC_SEQ_CST);
      if (at >= capacity) continue;
      int32_t* row = out + (size_t)at * 8;
      row[0] = (int32_t)blockIdx.x; row[1] = ti.group; row[2] = ti.row0; row[3] = ti.rows_valid;
      row[4] = ti.n0; row[5] = ti.num_kb; row[6] = ti.krow0; row[7] = ti.kcnt;
    }
  });
}

extern "C" void walk_tiles(int kind, int epi, int pair, int unit_walk, int num_groups, int N, int K,
                           int Mw, int n_tiles, int m_tiles, const int32_t* group_offs,
                           const int32_t* mtile_group, const int32_t* mtile_row0,
                           const int32_t* num_mtiles, int grid, int32_t* out, int32_t* count,
                           int capacity) {
  GemmParams p = {};
  p.kind = kind; p.epi = epi; p.pair = pair; p.unit_walk = unit_walk; p.num_groups = num_groups;
  p.N = N; p.K = K; p.Mw = Mw; p.n_tiles = n_tiles; p.m_tiles = m_tiles;
  p.group_offs = group_offs; p.mtile_group = mtile_group; p.mtile_row0 = mtile_row0;
  p.num_mtiles = num_mtiles;
  if (pair) walk<true>(p, grid, out, count, capacity);
  else walk<false>(p, grid, out, count, capacity);
}
"""


def cut(text: str, start: str, end: str = "\n}\n") -> str:
    i = text.index(start)
    i = text.rfind("\n", 0, i) + 1
    j = text.index(end, i) + len(end)
    return text[i:j]


@pytest.fixture(scope="module")
def walker(tmp_path_factory):
    from cuda_on_threads.host_build import compile_for_host
    gemm = (CSRC / "gemm_sm100.cuh").read_text()
    common = (CSRC / "common.cuh").read_text()
    skinny = (CSRC / "gemm_skinny_sm100.cuh").read_text()
    constants = "\n".join(re.findall(r"^constexpr int kBlock[MNK] = \d+;$", gemm, re.M)) + "\n" + \
        "\n".join(cut(gemm, f"enum {name} ", ";\n") for name in ("GemmKind", "EpiMode"))
    cursor = (cut(gemm, "struct TileCursor {", "\n};\n") + cut(gemm, "void cursor_load_unit(")
              + cut(gemm, "TileInfo cursor_tile(")
              + cut(gemm, "template <bool kPair>\n__device__ __forceinline__ TileCursor cursor_begin(")
              + cut(gemm, "void cursor_next("))
    src = HARNESS % dict(
        tile_info=cut(common, "struct TileInfo {", "\n};\n"),
        constants=constants,
        params=cut(gemm, "struct GemmParams {", "\n};\n"),
        total_tiles=cut(gemm, "int32_t total_tiles("),
        decode_tile=cut(gemm, "TileInfo decode_tile("),
        cursor=cursor,
        skinny=("constexpr int kSkinnyRows = 256;\n" + cut(skinny, "struct SkinnyTile {", "\n};\n")
                + cut(skinny, "SkinnyTile skinny_tile(") + cut(skinny, "int32_t skinny_half_col(")),
    )
    d = tmp_path_factory.mktemp("tile_walk")
    (d / "tile_walk.cpp").write_text(src)
    lib = C.CDLL(str(compile_for_host(d / "tile_walk.cpp", d / "libtilewalk.so")))
    lib.walk_tiles.restype = None
    lib.walk_skinny.restype = None
    return lib


def p(a):
    return C.c_void_p(a.ctypes.data)


def run(walker, *, kind, epi, pair, unit_walk, counts, N=0, K=0, Mw=0, grid):
    counts = np.asarray(counts, np.int64)
    groups = counts.size
    offs = np.r_[0, counts.cumsum()].astype(np.int32)
    tile_rows = 256 if pair else 128
    mg, mr = [], []
    for g in range(groups):
        for r0 in range(0, int(counts[g]), tile_rows):
            mg.append(g)
            mr.append(int(offs[g]) + r0)
    mtile_group = np.asarray(mg + [0], np.int32)
    mtile_row0 = np.asarray(mr + [0], np.int32)
    num_mtiles = np.asarray([len(mg)], np.int32)
    if kind == 0:
        n_tiles = -(-N // (128 if epi == 1 else 256))
        m_tiles = 0
        total = len(mg) * n_tiles
    else:
        n_tiles = -(-N // 256)
        m_tiles = -(-Mw // tile_rows)
        total = groups * m_tiles * n_tiles
    capacity = total * (2 if pair else 1) + 8
    out = np.full((capacity, 8), -1, np.int32)
    count = np.zeros(1, np.int32)
    walker.walk_tiles(kind, epi, int(pair), int(unit_walk), groups, N, K, Mw, n_tiles, m_tiles,
                      p(offs), p(mtile_group), p(mtile_row0), p(num_mtiles), grid, p(out), p(count),
                      capacity)
    assert count[0] <= capacity
    return out[:count[0]], offs, total


RAGGED = [  # rows per group, N, K
    ([146] * 7, 4096, 7168), ([0, 1, 128, 129, 0, 0, 300, 2000, 0], 7168, 2048),
    ([1170, 1170, 1171], 768, 192), ([0, 0, 0], 256, 64), ([5], 256, 64),
    ([256, 255, 257, 512, 0, 384], 1536, 4096),
]


@pytest.mark.parametrize("counts, N, K", RAGGED)
@pytest.mark.parametrize("pair, epi", [(False, 0), (False, 1), (True, 0), (False, 2)])
@pytest.mark.parametrize("grid", [1, 7, 148])
def test_ragged_row_tiles_are_walked_exactly_once(walker, counts, N, K, pair, epi, grid):
    if pair:
        grid = max(2, grid - grid % 2)           # clusters of two CTAs
    tiles, offs, total = run(walker, kind=0, epi=epi, pair=pair, unit_walk=False, counts=counts,
                             N=N, K=K, grid=grid)
    tile_rows = 256 if pair else 128
    ncols = 128 if epi == 1 else 256
    want = set()
    for g, c in enumerate(counts):
        for r0 in range(0, c, tile_rows):
            for n0 in range(0, N, ncols):
                for half in range(2 if pair else 1):
                    row0 = int(offs[g]) + r0 + half * 128
                    valid = max(0, min(128, int(offs[g + 1]) - row0))
                    want.add((g, row0, valid, n0, -(-K // 64), 0, 0))
    got = [tuple(int(v) for v in t[1:]) for t in tiles]
    assert len(got) == len(set(got)) == total * (2 if pair else 1)
    assert set(got) == want
    if pair:
        # both CTAs of a cluster take the same tiles, rank 0 the upper 128 rows
        by_cta = {}
        for t in tiles:
            by_cta.setdefault(int(t[0]), []).append(tuple(int(v) for v in t[1:]))
        for cta in range(0, grid, 2):
            a, b = by_cta.get(cta, []), by_cta.get(cta + 1, [])
            assert [(g, n0) for g, _, _, n0, *_ in a] == [(g, n0) for g, _, _, n0, *_ in b]
            assert all(y[1] == x[1] + 128 for x, y in zip(a, b))


REDUCE = [  # reduction rows per group, Mw, N
    ([146] * 6, 7168, 4096), ([0, 1, 64, 65, 300, 0, 1170], 2048, 7168),
    ([12, 0, 0, 700], 128, 256), ([200] * 3, 384, 512),
]


@pytest.mark.parametrize("counts, Mw, N", REDUCE)
@pytest.mark.parametrize("pair, unit_walk", [(False, False), (False, True), (True, False)])
@pytest.mark.parametrize("grid", [1, 6, 148])
def test_reduction_tiles_are_walked_exactly_once(walker, counts, Mw, N, pair, unit_walk, grid):
    if pair:
        grid = max(2, grid - grid % 2)
    tiles, offs, total = run(walker, kind=1, epi=0, pair=pair, unit_walk=unit_walk, counts=counts,
                             N=N, Mw=Mw, grid=grid)
    tile_rows = 256 if pair else 128
    want = set()
    for g, c in enumerate(counts):
        for m0 in range(0, Mw, tile_rows):
            for n0 in range(0, N, 256):
                for half in range(2 if pair else 1):
                    row0 = m0 + half * 128
                    valid = max(0, min(128, Mw - row0))
                    want.add((g, row0, valid, n0, -(-c // 64), int(offs[g]), c))
    got = [tuple(int(v) for v in t[1:]) for t in tiles]
    assert len(got) == len(set(got)) == total * (2 if pair else 1)
    assert set(got) == want
    if unit_walk:
        # a CTA finishes all m-tiles of one (group, n-tile) before it moves on
        m_tiles = -(-Mw // 128)
        by_cta = {}
        for t in tiles:
            by_cta.setdefault(int(t[0]), []).append((int(t[1]), int(t[4])))
        for seq in by_cta.values():
            assert len(seq) % m_tiles == 0
            for i in range(0, len(seq), m_tiles):
                assert len(set(seq[i:i + m_tiles])) == 1


@pytest.mark.parametrize("counts", [[146] * 5, [0, 1, 16, 17, 255, 256, 257, 0, 600], [0, 0], [40]])
@pytest.mark.parametrize("epi, N, F", [(0, 7168, 0), (1, 2048, 2048), (2, 512, 0)])
@pytest.mark.parametrize("grid", [1, 5, 148])
def test_skinny_tiles_are_walked_exactly_once(walker, counts, epi, N, F, grid):
    counts = np.asarray(counts, np.int64)
    offs = np.r_[0, counts.cumsum()].astype(np.int32)
    mg, mr = [], []
    for g, c in enumerate(counts):
        for r0 in range(0, int(c), 256):
            mg.append(g)
            mr.append(int(offs[g]) + r0)
    ncols = 128 if epi == 1 else 256
    n_tiles = -(-N // ncols)
    total = len(mg) * n_tiles
    out = np.full((total + 8, 8), -1, np.int32)
    count = np.zeros(1, np.int32)
    mtile_group = np.asarray(mg + [0], np.int32)      # named: the call must not outlive them
    mtile_row0 = np.asarray(mr + [0], np.int32)
    num_mtiles = np.asarray([len(mg)], np.int32)
    walker.walk_skinny(epi, F, n_tiles, p(offs), p(mtile_group), p(mtile_row0), p(num_mtiles), grid,
                       p(out), p(count), total + 8)
    want = set()
    for g, r0 in zip(mg, mr):
        valid = min(256, int(offs[g + 1]) - r0)
        for n0 in range(0, N, ncols):
            halves = (n0, F + n0) if epi == 1 else (n0, n0 + 128)
            want.add((g, r0, valid, n0, (valid + 15) // 16 * 16, *halves))
    got = [tuple(int(v) for v in t[1:]) for t in out[:count[0]]]
    assert len(got) == len(set(got)) == total
    assert set(got) == want
