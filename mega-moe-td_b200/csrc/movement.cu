// HBM / NVLink bound kernels around the grouped GEMMs: dispatch (row push into the
// owning rank's receive buffer), top-k reduce (gather-sum of returned rows), the gated
// activation backward, and the cross-rank flag barrier.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "internal.h"

namespace mm {

__device__ __forceinline__ uint4 ld_nc_16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_16(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// ---------------------------------------------------------------------------------
// Dispatch: one warp per send row, 16 bytes per lane per step, four steps in flight.
// ---------------------------------------------------------------------------------
constexpr int kDispatchThreads = 256;

__global__ void __launch_bounds__(kDispatchThreads)
dispatch_rows_kernel(const uint8_t* __restrict__ src, int row_bytes,
                     const float* __restrict__ weights, const int32_t* __restrict__ send_token,
                     const int32_t* __restrict__ send_route, const int32_t* __restrict__ send_bucket,
                     const int32_t* __restrict__ send_bucket_starts,
                     const int32_t* __restrict__ send_bucket_dst_starts,
                     const int32_t* __restrict__ local_stats, int epr, int capacity_rows,
                     void* const* __restrict__ peer_rows, float* const* __restrict__ peer_weights) {
  const int n = local_stats[0];
  const int lane = threadIdx.x & 31;
  const int warps_per_block = kDispatchThreads / 32;
  const int chunks = row_bytes >> 4;
  for (int i = blockIdx.x * warps_per_block + (threadIdx.x >> 5); i < n;
       i += gridDim.x * warps_per_block) {
    const int b = send_bucket[i];
    const int dst_rank = b / epr;
    const int dst_row = send_bucket_dst_starts[b] + (i - send_bucket_starts[b]);
    if (dst_row >= capacity_rows) continue;  // overflow is reported by the metadata kernel
    const uint8_t* s = src + (size_t)send_token[i] * row_bytes;
    uint8_t* d = reinterpret_cast<uint8_t*>(peer_rows[dst_rank]) + (size_t)dst_row * row_bytes;
    int c = lane;
    for (; c + 96 < chunks; c += 128) {
      const uint4 v0 = ld_nc_16(s + (size_t)c * 16);
      const uint4 v1 = ld_nc_16(s + (size_t)(c + 32) * 16);
      const uint4 v2 = ld_nc_16(s + (size_t)(c + 64) * 16);
      const uint4 v3 = ld_nc_16(s + (size_t)(c + 96) * 16);
      st_16(d + (size_t)c * 16, v0);
      st_16(d + (size_t)(c + 32) * 16, v1);
      st_16(d + (size_t)(c + 64) * 16, v2);
      st_16(d + (size_t)(c + 96) * 16, v3);
    }
    for (; c < chunks; c += 32) st_16(d + (size_t)c * 16, ld_nc_16(s + (size_t)c * 16));
    if (weights != nullptr && lane == 0) peer_weights[dst_rank][dst_row] = weights[send_route[i]];
  }
}

// ---------------------------------------------------------------------------------
// Top-k reduce: out[t] = bf16(sum_j fp32(rows[route_to_send[t*k + j]])), slot order.
// One block per token; each thread owns 16-byte column chunks.
// ---------------------------------------------------------------------------------
constexpr int kReduceThreads = 256;
constexpr int kMaxTopK = 64;

__global__ void __launch_bounds__(kReduceThreads)
topk_reduce_kernel(const uint8_t* __restrict__ rows, int64_t ld_bytes,
                   const int32_t* __restrict__ route_to_send, int tokens, int top_k, int row_bytes,
                   uint8_t* __restrict__ out, const __nv_bfloat16* __restrict__ gate_in,
                   __nv_bfloat16* __restrict__ gate_out, float* __restrict__ gate_out_f32) {
  __shared__ int32_t idx[kMaxTopK];
  const int chunks = row_bytes >> 4;
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    __syncthreads();
    if (threadIdx.x < top_k) {
      const int32_t r = route_to_send[(size_t)t * top_k + threadIdx.x];
      idx[threadIdx.x] = r;
      if (gate_in != nullptr) {
        const __nv_bfloat16 g = r >= 0 ? gate_in[r] : __float2bfloat16(0.0f);
        gate_out[(size_t)t * top_k + threadIdx.x] = g;
        if (gate_out_f32 != nullptr) gate_out_f32[(size_t)t * top_k + threadIdx.x] = __bfloat162float(g);
      }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < chunks; c += kReduceThreads) {
      float acc[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
      for (int j = 0; j < top_k; ++j) {
        const int32_t r = idx[j];
        if (r < 0) continue;
        const uint4 v = ld_nc_16(rows + (size_t)r * ld_bytes + (size_t)c * 16);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          acc[2 * q] += __uint_as_float(u[q] << 16);
          acc[2 * q + 1] += __uint_as_float(u[q] & 0xffff0000u);
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      st_16(out + (size_t)t * row_bytes + (size_t)c * 16, o);
    }
  }
}

// ---------------------------------------------------------------------------------
// Gated-activation backward: one block per received row.
// ---------------------------------------------------------------------------------
constexpr int kSwigluBwdThreads = 256;

__device__ __forceinline__ void act_pair(float g, float u, int act, float beta, float lbeta,
                                         float clamp, float& act_g, float& dact_g, float& v,
                                         float& dv) {
  if (act == MM_ACT_SWIGLU) {
    const float s = 1.0f / (1.0f + __expf(-g));
    act_g = g * s;
    dact_g = act_g * (1.0f - s) + s;
    v = u;
    dv = 1.0f;
  } else if (act == MM_ACT_CLAMP_SWIGLU) {
    const float gc = fminf(g, clamp);
    const float uc = fminf(fmaxf(u, -clamp), clamp);
    const float s = 1.0f / (1.0f + __expf(-gc));
    act_g = gc * s;
    dact_g = (s + gc * s * (1.0f - s)) * (g <= clamp ? 1.0f : 0.0f);
    v = uc;
    dv = fabsf(u) <= clamp ? 1.0f : 0.0f;
  } else {
    const float t = tanhf(g / beta);
    const float s = 1.0f / (1.0f + __expf(-g));
    act_g = beta * t * s;
    dact_g = (1.0f - t * t) * s + beta * t * s * (1.0f - s);
    if (lbeta > 0.0f) {
      const float tu = tanhf(u / lbeta);
      v = lbeta * tu;
      dv = 1.0f - tu * tu;
    } else {
      v = u;
      dv = 1.0f;
    }
  }
}

// Saved FC1 rows come as bf16, fp16 (plain copy) or fp8 E4M3 with one fp32 scale per row and
// per `group_n` columns (MM_FC1_* in the header).  Elements 2i, 2i+1 of the row part that
// starts at column `col0`, as fp32.
template <int kFmt>
__device__ __forceinline__ float2 load_fc1_pair(const void* row, int col0, int i,
                                                const float* scale_row, int group_n) {
  const int col = col0 + 2 * i;
  if constexpr (kFmt == MM_FC1_BF16) {
    return __bfloat1622float2(reinterpret_cast<const __nv_bfloat162*>(row)[col >> 1]);
  } else if constexpr (kFmt == MM_FC1_FP16) {
    return __half22float2(reinterpret_cast<const __half2*>(row)[col >> 1]);
  } else {
    const __nv_fp8x2_storage_t q = reinterpret_cast<const __nv_fp8x2_storage_t*>(row)[col >> 1];
    const float2 v = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(q, __NV_E4M3)));
    const float sc = scale_row[col / group_n];
    return make_float2(v.x * sc, v.y * sc);
  }
}

template <int kFmt>
__global__ void __launch_bounds__(kSwigluBwdThreads)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ grad_act, int64_t ld_ga,
                  const uint8_t* __restrict__ fc1_out, int64_t fc1_row_bytes,
                  const float* __restrict__ fc1_scale, int group_n,
                  const __nv_bfloat16* __restrict__ row_scale, int ffn,
                  const int32_t* __restrict__ num_rows, int max_rows,
                  __nv_bfloat16* __restrict__ grad_fc1, int64_t ld_gf,
                  __nv_bfloat16* __restrict__ grad_scale, int act, float beta, float lbeta,
                  float clamp, const int32_t* __restrict__ row_dst_rank,
                  const int32_t* __restrict__ row_dst_pos, void* const* __restrict__ peer_gate) {
  __shared__ float red[kSwigluBwdThreads / 32];
  const int n = min(*num_rows, max_rows);
  const int pairs = ffn >> 1;
  const int groups = kFmt == MM_FC1_FP8 ? (2 * ffn) / group_n : 0;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const __nv_bfloat162* dc = reinterpret_cast<const __nv_bfloat162*>(grad_act + (size_t)row * ld_ga);
    const uint8_t* raw = fc1_out + (size_t)row * fc1_row_bytes;
    const float* srow = kFmt == MM_FC1_FP8 ? fc1_scale + (size_t)row * groups : nullptr;
    __nv_bfloat162* dg = reinterpret_cast<__nv_bfloat162*>(grad_fc1 + (size_t)row * ld_gf);
    __nv_bfloat162* du = reinterpret_cast<__nv_bfloat162*>(grad_fc1 + (size_t)row * ld_gf + ffn);
    const float sc = __bfloat162float(row_scale[row]);
    float part = 0.0f;
    for (int i = threadIdx.x; i < pairs; i += kSwigluBwdThreads) {
      const float2 c = __bfloat1622float2(dc[i]);
      const float2 g = load_fc1_pair<kFmt>(raw, 0, i, srow, group_n);
      const float2 u = load_fc1_pair<kFmt>(raw, ffn, i, srow, group_n);
      float a0, d0, v0, dv0, a1, d1, v1, dv1;
      act_pair(g.x, u.x, act, beta, lbeta, clamp, a0, d0, v0, dv0);
      act_pair(g.y, u.y, act, beta, lbeta, clamp, a1, d1, v1, dv1);
      dg[i] = __floats2bfloat162_rn(c.x * d0 * v0 * sc, c.y * d1 * v1 * sc);
      du[i] = __floats2bfloat162_rn(c.x * a0 * dv0 * sc, c.y * a1 * dv1 * sc);
      part += a0 * v0 * c.x + a1 * v1 * c.y;
    }
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) part += __shfl_xor_sync(0xffffffffu, part, k);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.0f;
      for (int k = 0; k < kSwigluBwdThreads / 32; ++k) s += red[k];
      const __nv_bfloat16 v = __float2bfloat16_rn(s);
      grad_scale[row] = v;
      if (peer_gate != nullptr) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peer_gate[row_dst_rank[row]]);
        dst[row_dst_pos[row]] = v;
      }
    }
  }
}

// Activation recompute of the backward (saved-recompute mode): the weighted activation rows
// from the saved FC1 rows and the saved bf16 routing weights; fp32 intermediates, bf16 store.
template <int kFmt>
__global__ void __launch_bounds__(kSwigluBwdThreads)
swiglu_recompute_kernel(const uint8_t* __restrict__ fc1_out, int64_t fc1_row_bytes,
                        const float* __restrict__ fc1_scale, int group_n,
                        const __nv_bfloat16* __restrict__ row_scale, int ffn,
                        const int32_t* __restrict__ num_rows, int max_rows,
                        __nv_bfloat16* __restrict__ act_out, int64_t ld_act, int act, float beta,
                        float lbeta, float clamp) {
  const int n = min(*num_rows, max_rows);
  const int pairs = ffn >> 1;
  const int groups = kFmt == MM_FC1_FP8 ? (2 * ffn) / group_n : 0;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const uint8_t* raw = fc1_out + (size_t)row * fc1_row_bytes;
    const float* srow = kFmt == MM_FC1_FP8 ? fc1_scale + (size_t)row * groups : nullptr;
    __nv_bfloat162* out = reinterpret_cast<__nv_bfloat162*>(act_out + (size_t)row * ld_act);
    const float sc = __bfloat162float(row_scale[row]);
    for (int i = threadIdx.x; i < pairs; i += kSwigluBwdThreads) {
      const float2 g = load_fc1_pair<kFmt>(raw, 0, i, srow, group_n);
      const float2 u = load_fc1_pair<kFmt>(raw, ffn, i, srow, group_n);
      float a0, d0, v0, dv0, a1, d1, v1, dv1;
      act_pair(g.x, u.x, act, beta, lbeta, clamp, a0, d0, v0, dv0);
      act_pair(g.y, u.y, act, beta, lbeta, clamp, a1, d1, v1, dv1);
      out[i] = __floats2bfloat162_rn(a0 * v0 * sc, a1 * v1 * sc);
    }
  }
}

// Saved-format conversion of the raw bf16 FC1 rows: fp16 copy, or fp8 E4M3 with one fp32
// scale per row and per `group_n` columns (scale = amax / 448; an all-zero group keeps
// q = 0 and the scale 1 / 448).  One warp per (row, group) for fp8, 8 warps per block.
constexpr int kFp8Max = 448;

__global__ void __launch_bounds__(256)
fc1_to_fp16_kernel(const __nv_bfloat16* __restrict__ raw, int64_t ld_raw, int cols,
                   const int32_t* __restrict__ num_rows, int max_rows, __half* __restrict__ out,
                   int64_t ld_out) {
  const int n = min(*num_rows, max_rows);
  const int pairs = cols >> 1;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(raw + (size_t)row * ld_raw);
    __half2* dst = reinterpret_cast<__half2*>(out + (size_t)row * ld_out);
    for (int i = threadIdx.x; i < pairs; i += blockDim.x)
      dst[i] = __float22half2_rn(__bfloat1622float2(src[i]));
  }
}

__global__ void __launch_bounds__(256)
fc1_to_fp8_kernel(const __nv_bfloat16* __restrict__ raw, int64_t ld_raw, int cols, int group_n,
                  const int32_t* __restrict__ num_rows, int max_rows, uint8_t* __restrict__ out,
                  int64_t ld_out, float* __restrict__ scale) {
  const int n = min(*num_rows, max_rows);
  const int groups = cols / group_n;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const __nv_bfloat16* src = raw + (size_t)row * ld_raw;
    uint8_t* dst = out + (size_t)row * ld_out;
    for (int g = warp; g < groups; g += warps) {
      const int c0 = g * group_n;
      float amax = 0.0f;
      for (int c = lane; c < group_n; c += 32) amax = fmaxf(amax, fabsf(__bfloat162float(src[c0 + c])));
#pragma unroll
      for (int k = 16; k > 0; k >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, k));
      const float safe = amax > 0.0f ? amax : 1.0f;
      const float inv = (float)kFp8Max / safe;
      for (int c = lane; c < group_n; c += 32) {
        const float x = __bfloat162float(src[c0 + c]) * inv;
        dst[c0 + c] = (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
      }
      if (lane == 0) scale[(size_t)row * groups + g] = safe / (float)kFp8Max;
    }
  }
}

// ---------------------------------------------------------------------------------
// Cross-rank barrier through flag words in symmetric memory.
// ---------------------------------------------------------------------------------
__global__ void rank_barrier_kernel(int32_t* const* __restrict__ peer_flags, int rank, int world,
                                    int epoch, int phase, StatusRecord* status) {
  const int s = threadIdx.x;
  if (s >= world) return;
  if (phase != 2) {
    // Make every earlier store of this GPU (issued by preceding kernels of the stream)
    // visible system-wide before the flag that announces them.
    __threadfence_system();
    int32_t* remote = peer_flags[s] + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  }
  if (phase == 1) return;
  const int32_t* mine = peer_flags[rank] + s;
  const uint64_t t0 = globaltimer_ns();
  int32_t seen;
  uint32_t spins = 0;
  while (true) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (seen >= epoch) break;
    if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
      report_status(status, kWaitTimeout, kSiteRankBarrier, s, epoch, seen);
      break;
    }
    __nanosleep(64);
  }
}

// ---------------------------------------------------------------------------------
// Count exchange: every rank stores its count row into slot `rank` of every rank's count
// cube (plain peer stores), flags the row with the launch's epoch and waits (bounded) until
// all `world` rows of its own cube carry that epoch.  One block.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
count_exchange_kernel(const int32_t* __restrict__ count_row, int bins, int rank, int world,
                      int32_t* const* __restrict__ peer_cubes, int64_t cube_offset,
                      int32_t* const* __restrict__ peer_flags, const int32_t* my_flags, int epoch,
                      StatusRecord* status) {
  for (int i = threadIdx.x; i < world * bins; i += blockDim.x) {
    const int d = i / bins;
    const int b = i - d * bins;
    peer_cubes[d][cube_offset + (int64_t)rank * bins + b] = count_row[b];
  }
  // every thread's stores are visible system-wide before the flags that announce the row
  __threadfence_system();
  __syncthreads();
  for (int d = threadIdx.x; d < world; d += blockDim.x) {
    int32_t* flag = peer_flags[d] + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
  }
  for (int s = threadIdx.x; s < world; s += blockDim.x) {
    const int32_t* mine = my_flags + s;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    int32_t seen;
    while (true) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
      if (seen >= epoch) break;
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
        report_status(status, kWaitTimeout, kSiteCountFlag, s, epoch, seen);
        break;
      }
      __nanosleep(32);
    }
  }
}

}  // namespace mm

using namespace mm;

extern "C" {

int mm_count_exchange(const int32_t* count_row, int bins, int rank, int world,
                      int32_t* const* peer_cubes, int64_t cube_offset,
                      int32_t* const* peer_flags, const int32_t* my_flags, int epoch,
                      void* status, cudaStream_t stream) {
  if (!count_row || !peer_cubes || !peer_flags || !my_flags || bins <= 0 || world <= 0 ||
      rank < 0 || rank >= world || epoch <= 0 || cube_offset < 0) {
    set_error("mm_count_exchange: bad arguments");
    return MM_ERR_ARG;
  }
  count_exchange_kernel<<<1, 1024, 0, stream>>>(count_row, bins, rank, world, peer_cubes,
                                                cube_offset, peer_flags, my_flags, epoch,
                                                reinterpret_cast<StatusRecord*>(status));
  return check_launch("count_exchange_kernel");
}

int mm_dispatch_rows(const void* src, int hidden, const float* weights, const int32_t* send_token,
                     const int32_t* send_route, const int32_t* send_bucket,
                     const int32_t* send_bucket_starts, const int32_t* send_bucket_dst_starts,
                     const int32_t* local_stats, int max_routes, int epr, int capacity_rows,
                     void* const* peer_rows, float* const* peer_weights, cudaStream_t stream) {
  if (!src || !send_token || !send_route || !send_bucket || !send_bucket_starts ||
      !send_bucket_dst_starts || !local_stats || !peer_rows || (weights && !peer_weights)) {
    set_error("mm_dispatch_rows: null argument");
    return MM_ERR_ARG;
  }
  if (hidden <= 0 || (hidden % 8) || epr <= 0) {
    set_error("mm_dispatch_rows: hidden must be a positive multiple of 8 (got %d)", hidden);
    return MM_ERR_ARG;
  }
  if (max_routes <= 0) return MM_OK;
  int sms = 148;
  mm_num_sms(&sms);
  const int warps = kDispatchThreads / 32;
  int blocks = (max_routes + warps - 1) / warps;
  if (blocks > sms * 8) blocks = sms * 8;
  dispatch_rows_kernel<<<blocks, kDispatchThreads, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(src), hidden * 2, weights, send_token, send_route,
      send_bucket, send_bucket_starts, send_bucket_dst_starts, local_stats, epr, capacity_rows,
      peer_rows, peer_weights);
  return check_launch("dispatch_rows_kernel");
}

int mm_topk_reduce(const void* rows, int64_t ld_rows, const int32_t* route_to_send, int tokens,
                   int top_k, int hidden, void* out, const void* gate_in, void* gate_out,
                   float* gate_out_f32, cudaStream_t stream) {
  if (!rows || !route_to_send || !out || (gate_in && !gate_out)) {
    set_error("mm_topk_reduce: null argument");
    return MM_ERR_ARG;
  }
  if (top_k <= 0 || top_k > kMaxTopK || hidden <= 0 || (hidden % 8) || (ld_rows % 8)) {
    set_error("mm_topk_reduce: top_k must be in [1, %d] and hidden a multiple of 8", kMaxTopK);
    return MM_ERR_ARG;
  }
  if (tokens <= 0) return MM_OK;
  int sms = 148;
  mm_num_sms(&sms);
  int blocks = tokens < sms * 8 ? tokens : sms * 8;
  topk_reduce_kernel<<<blocks, kReduceThreads, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(rows), ld_rows * 2, route_to_send, tokens, top_k, hidden * 2,
      reinterpret_cast<uint8_t*>(out), reinterpret_cast<const __nv_bfloat16*>(gate_in),
      reinterpret_cast<__nv_bfloat16*>(gate_out), gate_out_f32);
  return check_launch("topk_reduce_kernel");
}

namespace {
int row_blocks(int max_rows) {
  int sms = 148;
  mm_num_sms(&sms);
  return max_rows < sms * 8 ? max_rows : sms * 8;
}

bool fc1_format_ok(int fmt, const void* scale, int group_n, int ffn, const char* who) {
  if (fmt != MM_FC1_BF16 && fmt != MM_FC1_FP16 && fmt != MM_FC1_FP8) {
    set_error("%s: unknown saved FC1 format %d", who, fmt);
    return false;
  }
  if (fmt == MM_FC1_FP8 && (!scale || group_n <= 0 || (group_n % 2) || ((2 * ffn) % group_n))) {
    set_error("%s: fp8 rows need a scale table and a group size that divides 2F", who);
    return false;
  }
  return true;
}

int64_t fc1_elem_bytes(int fmt) { return fmt == MM_FC1_FP8 ? 1 : 2; }
}  // namespace

int mm_swiglu_bwd(const void* grad_act, int64_t ld_ga, const void* fc1_out, int64_t ld_fc1,
                  const void* row_scale_bf16, int ffn, const int32_t* num_rows, int max_rows,
                  void* grad_fc1, int64_t ld_gf, void* grad_scale, int activation, float beta,
                  float linear_beta, float clamp_limit, const int32_t* row_dst_rank,
                  const int32_t* row_dst_pos, void* const* peer_gate, int fc1_format,
                  const float* fc1_scale, int fc1_scale_group, cudaStream_t stream) {
  if (!grad_act || !fc1_out || !row_scale_bf16 || !num_rows || !grad_fc1 || !grad_scale ||
      (peer_gate && (!row_dst_rank || !row_dst_pos))) {
    set_error("mm_swiglu_bwd: null argument");
    return MM_ERR_ARG;
  }
  if (ffn <= 0 || (ffn % 2) || (ld_ga % 2) || (ld_fc1 % 2) || (ld_gf % 2)) {
    set_error("mm_swiglu_bwd: ffn and leading dimensions must be even");
    return MM_ERR_ARG;
  }
  if (!fc1_format_ok(fc1_format, fc1_scale, fc1_scale_group, ffn, "mm_swiglu_bwd")) return MM_ERR_ARG;
  if (max_rows <= 0) return MM_OK;
  const int blocks = row_blocks(max_rows);
  const int64_t row_bytes = ld_fc1 * fc1_elem_bytes(fc1_format);
#define MM_LAUNCH_SWIGLU_BWD(FMT)                                                                  \
  swiglu_bwd_kernel<FMT><<<blocks, kSwigluBwdThreads, 0, stream>>>(                                \
      reinterpret_cast<const __nv_bfloat16*>(grad_act), ld_ga,                                     \
      reinterpret_cast<const uint8_t*>(fc1_out), row_bytes, fc1_scale, fc1_scale_group,            \
      reinterpret_cast<const __nv_bfloat16*>(row_scale_bf16), ffn, num_rows, max_rows,             \
      reinterpret_cast<__nv_bfloat16*>(grad_fc1), ld_gf, reinterpret_cast<__nv_bfloat16*>(grad_scale), \
      activation, beta, linear_beta, clamp_limit, row_dst_rank, row_dst_pos, peer_gate)
  if (fc1_format == MM_FC1_BF16) MM_LAUNCH_SWIGLU_BWD(MM_FC1_BF16);
  else if (fc1_format == MM_FC1_FP16) MM_LAUNCH_SWIGLU_BWD(MM_FC1_FP16);
  else MM_LAUNCH_SWIGLU_BWD(MM_FC1_FP8);
#undef MM_LAUNCH_SWIGLU_BWD
  return check_launch("swiglu_bwd_kernel");
}

int mm_swiglu_recompute(const void* fc1_out, int64_t ld_fc1, int fc1_format, const float* fc1_scale,
                        int fc1_scale_group, const void* row_scale_bf16, int ffn,
                        const int32_t* num_rows, int max_rows, void* act_out, int64_t ld_act,
                        int activation, float beta, float linear_beta, float clamp_limit,
                        cudaStream_t stream) {
  if (!fc1_out || !row_scale_bf16 || !num_rows || !act_out) {
    set_error("mm_swiglu_recompute: null argument");
    return MM_ERR_ARG;
  }
  if (ffn <= 0 || (ffn % 2) || (ld_fc1 % 2) || (ld_act % 2)) {
    set_error("mm_swiglu_recompute: ffn and leading dimensions must be even");
    return MM_ERR_ARG;
  }
  if (!fc1_format_ok(fc1_format, fc1_scale, fc1_scale_group, ffn, "mm_swiglu_recompute"))
    return MM_ERR_ARG;
  if (max_rows <= 0) return MM_OK;
  const int blocks = row_blocks(max_rows);
  const int64_t row_bytes = ld_fc1 * fc1_elem_bytes(fc1_format);
#define MM_LAUNCH_RECOMPUTE(FMT)                                                                   \
  swiglu_recompute_kernel<FMT><<<blocks, kSwigluBwdThreads, 0, stream>>>(                          \
      reinterpret_cast<const uint8_t*>(fc1_out), row_bytes, fc1_scale, fc1_scale_group,            \
      reinterpret_cast<const __nv_bfloat16*>(row_scale_bf16), ffn, num_rows, max_rows,             \
      reinterpret_cast<__nv_bfloat16*>(act_out), ld_act, activation, beta, linear_beta, clamp_limit)
  if (fc1_format == MM_FC1_BF16) MM_LAUNCH_RECOMPUTE(MM_FC1_BF16);
  else if (fc1_format == MM_FC1_FP16) MM_LAUNCH_RECOMPUTE(MM_FC1_FP16);
  else MM_LAUNCH_RECOMPUTE(MM_FC1_FP8);
#undef MM_LAUNCH_RECOMPUTE
  return check_launch("swiglu_recompute_kernel");
}

int mm_fc1_save_convert(const void* raw_bf16, int64_t ld_raw, int cols, const int32_t* num_rows,
                        int max_rows, int fc1_format, int scale_group, void* out, int64_t ld_out,
                        float* scale, cudaStream_t stream) {
  if (!raw_bf16 || !num_rows || !out) {
    set_error("mm_fc1_save_convert: null argument");
    return MM_ERR_ARG;
  }
  if (cols <= 0 || (cols % 2) || (ld_raw % 2) || (ld_out % 2)) {
    set_error("mm_fc1_save_convert: column count and leading dimensions must be even");
    return MM_ERR_ARG;
  }
  if (fc1_format == MM_FC1_FP8 && (!scale || scale_group <= 0 || (cols % scale_group))) {
    set_error("mm_fc1_save_convert: fp8 needs a scale table and a group size that divides the columns");
    return MM_ERR_ARG;
  }
  if (fc1_format != MM_FC1_FP8 && fc1_format != MM_FC1_FP16) {
    set_error("mm_fc1_save_convert: the target format must be fp16 or fp8");
    return MM_ERR_ARG;
  }
  if (max_rows <= 0) return MM_OK;
  const int blocks = row_blocks(max_rows);
  if (fc1_format == MM_FC1_FP16) {
    fc1_to_fp16_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(raw_bf16),
                                                   ld_raw, cols, num_rows, max_rows,
                                                   reinterpret_cast<__half*>(out), ld_out);
  } else {
    fc1_to_fp8_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(raw_bf16),
                                                  ld_raw, cols, scale_group, num_rows, max_rows,
                                                  reinterpret_cast<uint8_t*>(out), ld_out, scale);
  }
  return check_launch("fc1_save_convert");
}

int mm_rank_barrier(int32_t* const* peer_flags, int rank, int world, int epoch, int phase,
                    void* status, cudaStream_t stream) {
  if (!peer_flags || world <= 0 || world > 1024 || rank < 0 || rank >= world || phase < 0 ||
      phase > 2) {
    set_error("mm_rank_barrier: bad arguments");
    return MM_ERR_ARG;
  }
  rank_barrier_kernel<<<1, ((world + 31) / 32) * 32, 0, stream>>>(
      peer_flags, rank, world, epoch, phase, reinterpret_cast<StatusRecord*>(status));
  return check_launch("rank_barrier_kernel");
}

}  // extern "C"
