// Grouped GEMM for groups with few rows (sm_100a): the product is computed transposed.
//
// With ~150 rows per expert a 128-row output tile wastes most of its second row tile and the
// expert's weights are pulled into shared memory once per row tile.  Here the weight tile is the
// tensor core's M operand (128 output columns per MMA, two such halves per CTA tile) and the
// group's rows are the N operand, whose extent the instruction takes in steps of 16:
//
//     D[c, r] = sum_k W_g[k, c] * A[r, k]        c: 2 x 128 output columns, r: <= 256 rows
//
// so an expert with 146 rows costs MMAs of N = 160 and its weights cross the SM boundary once.
// TMEM holds the two halves (columns 0.. and 256..); a lane is an output column, a TMEM column
// a row, and the epilogue stores two-byte elements that are contiguous across the lanes of a
// warp.  The accumulator is not double-buffered: the reduction is long (K >= 2048) against an
// epilogue of a few thousand clocks.
//
// Roles as in grouped_gemm_kernel: warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 epilogue,
// warps 6..7 dispatch warps of a fused launch.  Row tiles come from the 256-row tile table.
#pragma once

#include "gemm_sm100.cuh"

namespace mm {

constexpr int kSkinnyStages = 3;
constexpr int kSkinnyRows = 256;                                  // rows of one tile (MMA N limit)
constexpr int kSkinnyHalfBytes = 128 * kBlockK * 2;               // 16 KB: 128 weight columns
constexpr int kSkinnyRowBoxRows = 32;                             // rows per TMA box of A
constexpr int kSkinnyRowBoxBytes = kSkinnyRowBoxRows * kBlockK * 2;  // 4 KB
constexpr int kSkinnyStageBytes = 2 * kSkinnyHalfBytes + kSkinnyRows * kBlockK * 2;  // 64 KB
static_assert(kSkinnyStages * kSkinnyStageBytes <= kStages * kStageBytes + kEpiWarps * kStagingPerWarp,
              "the skinny ring must fit the shared memory the launch already requests");

struct SkinnyTile {
  int32_t group;
  int32_t row0;        // first row (into A and the output)
  int32_t rows_valid;  // 1..256
  int32_t ntok;        // rows_valid rounded up to the MMA's step of 16
  int32_t n0;          // first output column of half 0 (kEpiSwiglu: first F column)
};

__device__ __forceinline__ SkinnyTile skinny_tile(const GemmParams& p, int32_t t) {
  SkinnyTile ti;
  const int32_t u = t / p.n_tiles;
  const int32_t nt = t - u * p.n_tiles;
  ti.group = p.mtile_group[u];
  ti.row0 = p.mtile_row0[u];
  const int32_t end = p.group_offs[ti.group + 1];
  ti.rows_valid = max(1, min(kSkinnyRows, end - ti.row0));
  ti.ntok = (ti.rows_valid + 15) & ~15;
  ti.n0 = nt * (p.epi == kEpiSwiglu ? 128 : 256);
  return ti;
}

// First weight column of half h of the tile.
__device__ __forceinline__ int32_t skinny_half_col(const GemmParams& p, const SkinnyTile& ti, int h) {
  if (p.epi == kEpiSwiglu) return (h ? p.swiglu_F : 0) + ti.n0;
  return ti.n0 + 128 * h;
}

// tmA: rows [rows_cap, K], box {64 k, 32 rows}.  tmB: the group's weights, MN-major
// ([K, N_total], box {64 n, 64 k, 1}) or K-major ([N_total, K], box {64 k, 128 n, 1}).
__global__ void __launch_bounds__(kGemmThreads, 1)
skinny_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stages = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kEpiWarps * kStagingPerWarp);
  uint64_t* full_bar = bars;                       // [kSkinnyStages]
  uint64_t* empty_bar = bars + kSkinnyStages;      // [kSkinnyStages]
  uint64_t* tmem_full = bars + 2 * kSkinnyStages;  // [1]
  uint64_t* tmem_empty = tmem_full + 1;            // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSkinnyStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, kEpiWarps);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int32_t ntiles = (*p.num_mtiles) * p.n_tiles;
  const int32_t num_kb = (p.K + kBlockK - 1) / kBlockK;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      int32_t ready_group = -1;
      // L2 prefetch cursor: runs p.prefetch_kb k-blocks ahead of the loads, across tiles, and
      // asks only for the weights (the group's rows are small and stay in L2 anyway).  The
      // requests do not wait for the dispatch flags, the weights are always there.
      int32_t pf_t = blockIdx.x;
      int32_t pf_kb = 0;
      int32_t pf_ahead = 0;   // k-blocks between the load cursor and the prefetch cursor
      SkinnyTile pf_ti = {};
      if (pf_t < ntiles) pf_ti = skinny_tile(p, pf_t);
      auto prefetch_step = [&]() {
        if (pf_t >= ntiles) return;
        const int32_t k0 = pf_kb * kBlockK;
        const int32_t c0 = skinny_half_col(p, pf_ti, 0);
        const int32_t c1 = skinny_half_col(p, pf_ti, 1);
        if (p.b_mn) {
          tma_prefetch_l2_3d(&tmB, c0, k0, pf_ti.group);
          tma_prefetch_l2_3d(&tmB, c0 + 64, k0, pf_ti.group);
          tma_prefetch_l2_3d(&tmB, c1, k0, pf_ti.group);
          tma_prefetch_l2_3d(&tmB, c1 + 64, k0, pf_ti.group);
        } else {
          tma_prefetch_l2_3d(&tmB, k0, c0, pf_ti.group);
          tma_prefetch_l2_3d(&tmB, k0, c1, pf_ti.group);
        }
        if (++pf_kb == num_kb) {
          pf_kb = 0;
          pf_t += gridDim.x;
          if (pf_t < ntiles) pf_ti = skinny_tile(p, pf_t);
        }
      };
      for (; pf_ahead < p.prefetch_kb; ++pf_ahead) prefetch_step();
      for (int32_t t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
        const SkinnyTile ti = skinny_tile(p, t);
        if (p.disp_src != nullptr && ti.group != ready_group) {
          if (!wait_expert_arrival(p, ti.group, abort_flag)) {
            alive = false;
            break;
          }
          ready_group = ti.group;
        }
        const int32_t nbox = (ti.ntok + kSkinnyRowBoxRows - 1) / kSkinnyRowBoxRows;
        const uint32_t bytes = 2 * kSkinnyHalfBytes + nbox * kSkinnyRowBoxBytes;
        const int32_t col0 = skinny_half_col(p, ti, 0);
        const int32_t col1 = skinny_half_col(p, ti, 1);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kSiteSmemEmpty, stage)) {
            alive = false;
            break;
          }
          if (p.prefetch_kb > 0) prefetch_step();   // keeps the cursor prefetch_kb blocks ahead
          uint8_t* sW = stages + stage * kSkinnyStageBytes;
          uint8_t* sX = sW + 2 * kSkinnyHalfBytes;
          uint64_t* fb = &full_bar[stage];
          mbar_arrive_expect_tx(fb, bytes);
          const int32_t k0 = kb * kBlockK;
          if (p.b_mn) {
            tma_load_3d(sW, &tmB, fb, col0, k0, ti.group);
            tma_load_3d(sW + kBoxBytes, &tmB, fb, col0 + 64, k0, ti.group);
            tma_load_3d(sW + kSkinnyHalfBytes, &tmB, fb, col1, k0, ti.group);
            tma_load_3d(sW + kSkinnyHalfBytes + kBoxBytes, &tmB, fb, col1 + 64, k0, ti.group);
          } else {
            tma_load_3d(sW, &tmB, fb, k0, col0, ti.group);
            tma_load_3d(sW + kSkinnyHalfBytes, &tmB, fb, k0, col1, ti.group);
          }
          for (int32_t b = 0; b < nbox; ++b)
            tma_load_2d(sX + b * kSkinnyRowBoxBytes, &tmA, fb, k0, ti.row0 + b * kSkinnyRowBoxRows);
          if (++stage == kSkinnyStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!alive) {
        // Give loads already in flight time to land before the CTA retires.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 1000000ull) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    // One lane runs the loop alone: every clock between two MMA issues idles the tensor pipe.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      const uint32_t w_lbo = p.b_mn ? (uint32_t)kBoxBytes : 16u;
      const uint32_t w_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
      for (int32_t t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
        const SkinnyTile ti = skinny_tile(p, t);
        if (!mbar_wait(tmem_empty, acc_phase ^ 1, abort_flag, p.status, kSiteTmemEmpty, 0)) break;
        tc_fence_after_sync();
        const uint32_t idesc = make_idesc_bf16(128, ti.ntok, p.b_mn, 0);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kSiteSmemFull, stage)) {
            alive = false;
            break;
          }
          tc_fence_after_sync();
#ifdef MM_PROFILE
          if (p.prof_skip_mma) {
            mbar_arrive(&empty_bar[stage]);
          } else
#endif
          {
            const uint32_t w_addr = smem_u32(stages + stage * kSkinnyStageBytes);
            const uint64_t w0_desc = make_smem_desc(w_addr, w_lbo, 1024);
            const uint64_t w1_desc = make_smem_desc(w_addr + kSkinnyHalfBytes, w_lbo, 1024);
            const uint64_t x_desc = make_smem_desc(w_addr + 2 * kSkinnyHalfBytes, 16u, 1024);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              const uint32_t accumulate = (kb | k) != 0 ? 1u : 0u;
              umma_f16(tmem_base, w0_desc + (uint64_t)(k * w_kstep), x_desc + (uint64_t)(k * 2),
                       idesc, accumulate);
              umma_f16(tmem_base + 256, w1_desc + (uint64_t)(k * w_kstep),
                       x_desc + (uint64_t)(k * 2), idesc, accumulate);
            }
            umma_commit(&empty_bar[stage]);
          }
          if (++stage == kSkinnyStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!alive) break;
#ifdef MM_PROFILE
        if (p.prof_skip_mma) {
          mbar_arrive(tmem_full);
        } else
#endif
        umma_commit(tmem_full);
        acc_phase ^= 1;
      }
    }
  } else if (warp >= 2 + kEpiWarps) {
    // ----------------------------- dispatch warps -----------------------------
    dispatch_warp_run(p, (int32_t)(warp - 2 - kEpiWarps), lane);
  } else {
    // -------------------------------- epilogue --------------------------------
    const uint32_t q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t acc_phase = 0;
    for (int32_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
      const SkinnyTile ti = skinny_tile(p, t);
      // Destination lookups do not depend on the accumulator: resolve them while the main loop
      // of this tile is still running.  Lane l owns row j * 32 + l of every 32-row chunk j.
      // (The routing weights of a fused launch arrive with the dispatched rows, so they are
      // read only after the accumulator is complete.)
      constexpr int kMaxChunks = kSkinnyRows / 32;
      const int32_t nchunks = (ti.rows_valid + 31) >> 5;
      __nv_bfloat16* my_ptr[kMaxChunks];
#pragma unroll
      for (int j = 0; j < kMaxChunks; ++j) {
        my_ptr[j] = nullptr;
        const int32_t r = j * 32 + (int32_t)lane;
        if (r < ti.rows_valid) {
          const int32_t row = ti.row0 + r;
          if (p.epi == kEpiSwiglu) {
            // routing weights: see below
          } else if (p.epi == kEpiScatter) {
            my_ptr[j] = p.peer_bases[p.row_dst_rank[row]] + (int64_t)p.row_dst_pos[row] * p.ld_dst;
          } else {
            my_ptr[j] = p.out + (int64_t)row * p.ld_out;
          }
        }
      }
      if (!mbar_wait(tmem_full, acc_phase, abort_flag, p.status, kSiteTmemFull, 0)) break;
      tc_fence_after_sync();
      const uint32_t t_acc = tmem_base + ((q * 32u) << 16);
      const int32_t lane_col = (int32_t)(q * 32 + lane);   // output column inside a half

      if (p.epi == kEpiSwiglu) {
        const int32_t f = ti.n0 + lane_col;                 // column of act, gate column of raw
        // the chunk loop stays rolled (its body is large); the next chunk's routing weights are
        // fetched while this chunk is converted
        float w_next = (int32_t)lane < ti.rows_valid ? p.row_weight[ti.row0 + (int32_t)lane] : 0.0f;
#pragma unroll 1
        for (int j = 0; j < nchunks; ++j) {
          const float w_mine = w_next;
          if (q == 0 && ti.n0 == 0 && p.row_weight_bf16 != nullptr &&
              j * 32 + (int32_t)lane < ti.rows_valid)
            p.row_weight_bf16[ti.row0 + j * 32 + (int32_t)lane] = __float2bfloat16_rn(w_mine);
          const int32_t rn = (j + 1) * 32 + (int32_t)lane;
          w_next = rn < ti.rows_valid ? p.row_weight[ti.row0 + rn] : 0.0f;
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_acc + j * 32, rg);
          tmem_ld_32x32(t_acc + 256 + j * 32, ru);
          tmem_ld_wait_regs(rg);
          tmem_ld_wait_regs(ru);
          const int32_t cnt = min(32, ti.rows_valid - j * 32);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float w = __shfl_sync(0xffffffffu, w_mine, i);
            if (i < cnt) {
              const int64_t row = (int64_t)ti.row0 + j * 32 + i;
              const float g = bf16_round(__uint_as_float(rg[i]));
              const float u = bf16_round(__uint_as_float(ru[i]));
              p.out[row * p.ld_out + f] = __float2bfloat16(gated_activation(g, u, p) * w);
              if (p.out2 != nullptr) {
                p.out2[row * p.ld_out2 + f] = __float2bfloat16(g);
                p.out2[row * p.ld_out2 + p.swiglu_F + f] = __float2bfloat16(u);
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          const int32_t c = ti.n0 + 128 * h + lane_col;
          if (ti.n0 + 128 * h >= p.N) break;
          const bool col_ok = c < p.N;
#pragma unroll
          for (int j = 0; j < kMaxChunks; ++j) {
            if (j >= nchunks) break;
            uint32_t r[32];
            tmem_ld_32x32(t_acc + h * 256 + j * 32, r);
            tmem_ld_wait_regs(r);
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(
                  __shfl_sync(0xffffffffu, (unsigned long long)my_ptr[j], i));
              if (dst != nullptr && col_ok) dst[c] = __float2bfloat16(__uint_as_float(r[i]));
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty);
      acc_phase ^= 1;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Activation pass of the two-step FC1 (skinny mode): act[row, f] = activation(gate, up) * w[row]
// from the raw gate|up rows a plain GEMM stored as bf16 -- the same rounding points as the
// fused epilogue.  With few rows per expert the raw rows are a small fraction of the weight
// traffic, and the plain GEMM reads 256 contiguous weight columns per tile instead of two
// separate 128-column runs.  One block per row, 16-byte accesses; the number of rows is
// group_offs[num_groups].
constexpr int kSwigluRowsThreads = 256;

__global__ void __launch_bounds__(kSwigluRowsThreads)
swiglu_rows_kernel(const GemmParams p, const __nv_bfloat16* __restrict__ raw, int64_t ld_raw,
                   int32_t max_rows) {
  const int32_t n = min(p.group_offs[p.num_groups], max_rows);
  const int32_t chunks = p.swiglu_F >> 3;
  for (int32_t row = blockIdx.x; row < n; row += gridDim.x) {
    const uint4* gate = reinterpret_cast<const uint4*>(raw + (int64_t)row * ld_raw);
    const uint4* up = reinterpret_cast<const uint4*>(raw + (int64_t)row * ld_raw + p.swiglu_F);
    uint4* act = reinterpret_cast<uint4*>(p.out + (int64_t)row * p.ld_out);
    const float w = p.row_weight[row];
    if (threadIdx.x == 0 && p.row_weight_bf16 != nullptr)
      p.row_weight_bf16[row] = __float2bfloat16_rn(w);
    for (int32_t i = threadIdx.x; i < chunks; i += kSwigluRowsThreads) {
      const uint4 g4 = gate[i];
      const uint4 u4 = up[i];
      const uint32_t gs[4] = {g4.x, g4.y, g4.z, g4.w};
      const uint32_t us[4] = {u4.x, u4.y, u4.z, u4.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gs[k]));
        const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&us[k]));
        o[k] = pack_bf16x2(gated_activation(g.x, u.x, p) * w, gated_activation(g.y, u.y, p) * w);
      }
      act[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace mm
