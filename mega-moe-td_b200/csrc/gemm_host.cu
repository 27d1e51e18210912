// Host-side launchers of the tcgen05 grouped GEMM: tensor-map construction and the
// four C-ABI entry points that use it (declared in include/mega_moe_b200.h).
#include <cudaTypedefs.h>

#include <stdio.h>
#include <stdlib.h>

#include <mutex>

#include "gemm_skinny_sm100.cuh"
#include "internal.h"

namespace mm {

namespace {

PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
std::once_flag g_encode_once;

bool load_encode_fn() {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
  });
  return g_encode != nullptr;
}

// bf16 tensor map with a 128-byte swizzle; dims/strides innermost first, strides in bytes
// for dimensions 1.. (dimension 0 is contiguous).
bool encode_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box) {
  if (!load_encode_fn()) {
    set_error("cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bdim[5];
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank,
                        const_cast<void*>(base), gdim, gstr, bdim, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed (code %d): rank=%d dims=%llu,%llu box=%u,%u base=%p",
              (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0],
              box[1], base);
    return false;
  }
  return true;
}

PerDeviceOnce g_gemm_attr;

// Opt-in shared-memory size of the three GEMM kernels on the current device, and its SM count.
bool prepare_kernel(int* num_sms) {
  const int rc = g_gemm_attr([] {
    cudaError_t e = cudaFuncSetAttribute(grouped_gemm_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(grouped_gemm_kernel<true>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(skinny_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               kGemmSmemBytes);
    if (e != cudaSuccess) {
      set_error("cudaFuncSetAttribute(grouped_gemm_kernel): %s", cudaGetErrorString(e));
      return (int)MM_ERR_CUDA;
    }
    return (int)MM_OK;
  });
  if (rc != MM_OK) return false;
  return mm_num_sms(num_sms) == MM_OK;
}

#ifdef MM_PROFILE
unsigned long long* g_prof_buffer = nullptr;   // [grid, 16] counters of the next launches
#endif

int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
           const GemmParams& p_in, int grid_limit, cudaStream_t stream) {
  int num_sms = 0;
  if (!prepare_kernel(&num_sms)) return MM_ERR_CUDA;
  GemmParams p = p_in;
#ifdef MM_PROFILE
  p.prof = g_prof_buffer;
  p.prof_skip_mma = getenv("MM_PROFILE_SKIP_MMA") != nullptr;
#endif
  int grid = num_sms;
  if (grid_limit > 0 && grid_limit < grid) grid = grid_limit;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kGemmSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  cudaError_t e;
  if (p.pair) {
    // clusters of two CTAs: the grid must be even and no larger than what can be co-resident
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    static int max_pairs = -1;
    if (max_pairs < 0) {
      cudaLaunchConfig_t probe = cfg;
      probe.gridDim = dim3(num_sms & ~1, 1, 1);
      int n = 0;
      cudaError_t pe = cudaOccupancyMaxActiveClusters(&n, grouped_gemm_kernel<true>, &probe);
      if (pe != cudaSuccess || n <= 0) {
        set_error("cudaOccupancyMaxActiveClusters: %s (clusters=%d)", cudaGetErrorString(pe), n);
        return MM_ERR_CUDA;
      }
      max_pairs = n;
    }
    grid &= ~1;
    if (grid > 2 * max_pairs) grid = 2 * max_pairs;
    if (grid < 2) grid = 2;
    cfg.gridDim = dim3(grid, 1, 1);
    e = cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<true>, tmA, tmB, tmC, p);
  } else {
    cfg.gridDim = dim3(grid, 1, 1);
    e = cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<false>, tmA, tmB, tmC, p);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("grouped_gemm_kernel launch: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

// Transposed-product kernel for groups with few rows (tile mode 2).
int launch_skinny(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p_in,
                  int grid_limit, cudaStream_t stream) {
  int num_sms = 0;
  if (!prepare_kernel(&num_sms)) return MM_ERR_CUDA;
  GemmParams p = p_in;
#ifdef MM_PROFILE
  p.prof = nullptr;
  p.prof_skip_mma = getenv("MM_PROFILE_SKIP_MMA") != nullptr;
#endif
  int grid = num_sms;
  if (grid_limit > 0 && grid_limit < grid) grid = grid_limit;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.dynamicSmemBytes = kGemmSmemBytes;
  cfg.stream = stream;
  cudaError_t e = cudaLaunchKernelEx(&cfg, skinny_gemm_kernel, tmA, tmB, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("skinny_gemm_kernel launch: %s", cudaGetErrorString(e));
    return MM_ERR_CUDA;
  }
  return MM_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// A rows [a_rows_cap, K] (K contiguous, leading dimension lda elements).
// B per group: b_k_major != 0 -> [N_total, K] with K contiguous; else [K, N_total] with N contiguous.
bool fill_dispatch(const mm_dispatch_desc* x, GemmParams& p) {
  if (x == nullptr) return true;
  if (!x->src || !x->send_token || !x->send_route || !x->send_bucket_starts ||
      !x->send_bucket_dst_starts || !x->count_row || !x->order_prefix || !x->local_stats ||
      !x->bucket_done || !x->peer_rows || !x->peer_flags || !x->my_flags ||
      (x->weights && !x->peer_weights) || x->hidden <= 0 || (x->hidden % 8) || x->world <= 0 ||
      x->rank < 0 || x->rank >= x->world || x->epr <= 0 || x->epoch <= 0) {
    set_error("fused dispatch descriptor is incomplete or inconsistent");
    return false;
  }
  p.disp_src = reinterpret_cast<const uint8_t*>(x->src);
  p.disp_row_bytes = x->hidden * 2;
  p.disp_rank = x->rank;
  p.disp_world = x->world;
  p.disp_epr = x->epr;
  p.disp_capacity = x->capacity_rows;
  p.disp_epoch = x->epoch;
  p.disp_weights = x->weights;
  p.disp_send_token = x->send_token;
  p.disp_send_route = x->send_route;
  p.disp_bucket_starts = x->send_bucket_starts;
  p.disp_dst_starts = x->send_bucket_dst_starts;
  p.disp_counts = x->count_row;
  p.disp_order_prefix = x->order_prefix;
  p.disp_num_send = x->local_stats;
  p.disp_bucket_done = x->bucket_done;
  p.disp_peer_rows = x->peer_rows;
  p.disp_peer_weights = x->peer_weights;
  p.disp_peer_flags = x->peer_flags;
  p.disp_my_flags = x->my_flags;
  return true;
}

int grouped_rows_gemm(int epi, const mm_gemm_desc& d, GemmParams p, cudaStream_t stream) {
  if (!aligned16(d.a) || !aligned16(d.b) || (d.lda % 8) || (d.b_ld % 8) || (d.b_group_stride % 8)) {
    set_error("grouped GEMM operands must be 16-byte aligned with strides that are multiples of 8");
    return MM_ERR_ARG;
  }
  if (d.K <= 0 || (d.K % 8) || d.N <= 0 || (d.N % 32)) {
    set_error("grouped GEMM needs K %% 8 == 0 and N %% 32 == 0 (K=%d N=%d)", d.K, d.N);
    return MM_ERR_ARG;
  }
  if (d.pair < 0 || d.pair > 2) {
    set_error("grouped GEMM: tile mode %d is not one of 0 (single), 1 (pair), 2 (skinny)", d.pair);
    return MM_ERR_ARG;
  }
  const bool skinny = d.pair == 2;
  CUtensorMap tmA, tmB;
  {
    uint64_t dims[2] = {(uint64_t)d.K, (uint64_t)d.a_rows_cap};
    uint64_t str[1] = {(uint64_t)d.lda * 2};
    uint32_t box[2] = {64, (uint32_t)(skinny ? kSkinnyRowBoxRows : kBlockM)};
    if (!encode_map(&tmA, d.a, 2, dims, str, box)) return MM_ERR_CUDA;
  }
  const int b_cols = d.b_cols_total;  // full column extent of B (2F for the packed gate|up table)
  if (d.b_k_major) {
    uint64_t dims[3] = {(uint64_t)d.K, (uint64_t)b_cols, (uint64_t)d.num_groups};
    uint64_t str[2] = {(uint64_t)d.b_ld * 2, (uint64_t)d.b_group_stride * 2};
    uint32_t box[3] = {64, (uint32_t)(d.pair ? kBlockN / 2 : kBlockN), 1};  // 128 rows in modes 1, 2
    if (!encode_map(&tmB, d.b, 3, dims, str, box)) return MM_ERR_CUDA;
  } else if (!skinny && epi == kEpiSwiglu && d.pair == 0 && (d.N % 64) == 0 && b_cols == 2 * d.N) {
    // fused FC1 on one CTA: gate boxes and up boxes of a tile come with one instruction
    uint64_t dims[5] = {64, (uint64_t)d.K, (uint64_t)d.N / 64, 2, (uint64_t)d.num_groups};
    uint64_t str[4] = {(uint64_t)d.b_ld * 2, 128, (uint64_t)d.N * 2,
                       (uint64_t)d.b_group_stride * 2};
    uint32_t box[5] = {64, 64, 2, 2, 1};
    if (!encode_map(&tmB, d.b, 5, dims, str, box)) return MM_ERR_CUDA;
    p.b_multibox = 2;
  } else if (!skinny && (b_cols % 64) == 0 && !(epi == kEpiSwiglu && d.pair == 0)) {
    uint64_t dims[4] = {64, (uint64_t)d.K, (uint64_t)b_cols / 64, (uint64_t)d.num_groups};
    uint64_t str[3] = {(uint64_t)d.b_ld * 2, 128, (uint64_t)d.b_group_stride * 2};
    uint32_t box[4] = {64, 64, (uint32_t)(d.pair ? 2 : 4), 1};
    if (!encode_map(&tmB, d.b, 4, dims, str, box)) return MM_ERR_CUDA;
    p.b_multibox = 1;
  } else {
    uint64_t dims[3] = {(uint64_t)b_cols, (uint64_t)d.K, (uint64_t)d.num_groups};
    uint64_t str[2] = {(uint64_t)d.b_ld * 2, (uint64_t)d.b_group_stride * 2};
    uint32_t box[3] = {64, 64, 1};
    if (!encode_map(&tmB, d.b, 3, dims, str, box)) return MM_ERR_CUDA;
  }
  p.kind = kGroupedRows;
  p.epi = epi;
  p.num_groups = d.num_groups;
  p.N = d.N;
  p.K = d.K;
  p.a_mn = 0;
  p.b_mn = d.b_k_major ? 0 : 1;
  p.pair = d.pair == 1 ? 1 : 0;
  p.idesc = make_idesc_bf16(p.pair ? 2 * kBlockM : kBlockM, kBlockN, 0, p.b_mn);
  p.group_offs = d.group_offs;
  p.mtile_group = d.mtile_group;
  p.mtile_row0 = d.mtile_row0;
  p.num_mtiles = d.num_mtiles;
  p.status = reinterpret_cast<StatusRecord*>(d.status);
  if (epi == kEpiSwiglu) {
    if (d.b_k_major || (d.N % 128)) {
      set_error("fused FC1 needs the [E, H, 2F] weight layout and F %% 128 == 0");
      return MM_ERR_ARG;
    }
    p.n_tiles = d.N / (kBlockN / 2);
    p.swiglu_F = d.N;
  } else {
    p.n_tiles = (d.N + kBlockN - 1) / kBlockN;
    p.swiglu_F = 0;
  }
  p.tma_store = 0;
  if (skinny) {
    static const int prefetch_kb = [] {
      const char* env = getenv("MM_SKINNY_PREFETCH");   // k-blocks of L2 prefetch distance
      return env ? atoi(env) : 0;
    }();
    p.prefetch_kb = prefetch_kb < 0 ? 0 : (prefetch_kb > 64 ? 64 : prefetch_kb);
    return launch_skinny(tmA, tmB, p, d.grid_limit, stream);
  }
  return launch(tmA, tmB, tmA, p, d.grid_limit, stream);
}

}  // namespace mm

using namespace mm;

extern "C" {

int mm_fc1_swiglu(const mm_gemm_desc* d, const mm_dispatch_desc* dispatch, void* act_out,
                  int64_t ld_act, void* raw_out,
                  int64_t ld_raw, const float* row_weight, void* row_weight_bf16_out,
                  int activation, float beta, float linear_beta, float clamp_limit,
                  cudaStream_t stream) {
  if (!d || !act_out || !row_weight) {
    set_error("mm_fc1_swiglu: null argument");
    return MM_ERR_ARG;
  }
  GemmParams p{};
  p.out = reinterpret_cast<__nv_bfloat16*>(act_out);
  p.ld_out = ld_act;
  p.out2 = reinterpret_cast<__nv_bfloat16*>(raw_out);
  p.ld_out2 = ld_raw;
  p.row_weight = row_weight;
  p.row_weight_bf16 = reinterpret_cast<__nv_bfloat16*>(row_weight_bf16_out);
  p.act = activation;
  p.act_beta = beta;
  p.act_linear_beta = linear_beta;
  p.act_clamp = clamp_limit;
  if (!fill_dispatch(dispatch, p)) return MM_ERR_ARG;
  if (d->pair == 2 && raw_out != nullptr) {
    // Skinny mode with a raw buffer: a plain GEMM over all 2F columns stores the raw gate|up
    // rows, a row-wise pass applies the activation (see swiglu_rows_kernel).
    if ((d->N % 128) || (ld_raw % 8) || (ld_act % 8) || !aligned16(raw_out) || !aligned16(act_out)) {
      set_error("fused FC1 needs F %% 128 == 0 and 16-byte aligned outputs");
      return MM_ERR_ARG;
    }
    mm_gemm_desc wide = *d;
    wide.N = 2 * d->N;
    GemmParams g = p;
    g.out = reinterpret_cast<__nv_bfloat16*>(raw_out);
    g.ld_out = ld_raw;
    g.out2 = nullptr;
    g.row_weight_bf16 = nullptr;
    const int rc = grouped_rows_gemm(kEpiStore, wide, g, stream);
    if (rc != MM_OK) return rc;
    GemmParams a{};
    a.out = p.out;
    a.ld_out = p.ld_out;
    a.row_weight = row_weight;
    a.row_weight_bf16 = p.row_weight_bf16;
    a.act = activation;
    a.act_beta = beta;
    a.act_linear_beta = linear_beta;
    a.act_clamp = clamp_limit;
    a.swiglu_F = d->N;
    a.group_offs = d->group_offs;
    a.num_groups = d->num_groups;
    const int max_rows = (int)(d->a_rows_cap < (int64_t)INT32_MAX ? d->a_rows_cap : INT32_MAX);
    int sms = 148;
    mm_num_sms(&sms);
    int blocks = sms * 8;
    if (blocks > max_rows) blocks = max_rows;
    if (blocks < 1) blocks = 1;
    swiglu_rows_kernel<<<blocks, kSwigluRowsThreads, 0, stream>>>(
        a, reinterpret_cast<const __nv_bfloat16*>(raw_out), ld_raw, max_rows);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
      set_error("swiglu_rows_kernel launch: %s", cudaGetErrorString(e));
      return MM_ERR_CUDA;
    }
    return MM_OK;
  }
  return grouped_rows_gemm(kEpiSwiglu, *d, p, stream);
}

int mm_grouped_gemm(const mm_gemm_desc* d, const mm_dispatch_desc* dispatch, void* out,
                    int64_t ld_out, cudaStream_t stream) {
  if (!d || !out) {
    set_error("mm_grouped_gemm: null argument");
    return MM_ERR_ARG;
  }
  GemmParams p{};
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  if (!fill_dispatch(dispatch, p)) return MM_ERR_ARG;
  return grouped_rows_gemm(kEpiStore, *d, p, stream);
}

int mm_grouped_gemm_scatter(const mm_gemm_desc* d, const int32_t* row_dst_rank,
                            const int32_t* row_dst_pos, void* const* peer_bases, int64_t ld_dst,
                            cudaStream_t stream) {
  if (!d || !row_dst_rank || !row_dst_pos || !peer_bases) {
    set_error("mm_grouped_gemm_scatter: null argument");
    return MM_ERR_ARG;
  }
  GemmParams p{};
  p.row_dst_rank = row_dst_rank;
  p.row_dst_pos = row_dst_pos;
  p.peer_bases = reinterpret_cast<__nv_bfloat16* const*>(peer_bases);
  p.ld_dst = ld_dst;
  {
    const char* env = getenv("MM_SCATTER_WIDE");
    p.wide_store = (env == nullptr || env[0] != '0') ? 1 : 0;
  }
  return grouped_rows_gemm(kEpiScatter, *d, p, stream);
}

int mm_grouped_wgrad(const void* grad_out, int64_t ld_go, int32_t Mw, const void* orig_in,
                     int64_t ld_in, int32_t Nw, int64_t rows_cap, const int32_t* group_offs,
                     int32_t num_groups, void* out, int64_t ld_out, int64_t out_group_stride,
                     void* status, int32_t grid_limit, int32_t pair, cudaStream_t stream) {
  if (!grad_out || !orig_in || !group_offs || !out) {
    set_error("mm_grouped_wgrad: null argument");
    return MM_ERR_ARG;
  }
  if ((Mw % 8) || (Nw % 32) || (ld_go % 8) || (ld_in % 8) || (ld_out % 8) ||
      (out_group_stride % 8)) {
    set_error("mm_grouped_wgrad: extents/strides must be multiples of 8 (Nw of 32)");
    return MM_ERR_ARG;
  }
  CUtensorMap tmA, tmB, tmC;
  {
    uint64_t dims[3] = {(uint64_t)Nw, (uint64_t)Mw, (uint64_t)num_groups};
    uint64_t str[2] = {(uint64_t)ld_out * 2, (uint64_t)out_group_stride * 2};
    uint32_t box[3] = {64, 32, 1};
    if (!aligned16(out) || !encode_map(&tmC, out, 3, dims, str, box)) {
      if (aligned16(out)) return MM_ERR_CUDA;
      set_error("mm_grouped_wgrad: out must be 16-byte aligned");
      return MM_ERR_ARG;
    }
  }
  GemmParams p{};
  if ((Mw % 64) == 0) {
    uint64_t dims[3] = {64, (uint64_t)rows_cap, (uint64_t)Mw / 64};
    uint64_t str[2] = {(uint64_t)ld_go * 2, 128};
    uint32_t box[3] = {64, 64, 2};
    if (!encode_map(&tmA, grad_out, 3, dims, str, box)) return MM_ERR_CUDA;
    p.a_multibox = 1;
  } else {
    uint64_t dims[2] = {(uint64_t)Mw, (uint64_t)rows_cap};
    uint64_t str[1] = {(uint64_t)ld_go * 2};
    uint32_t box[2] = {64, 64};
    if (!encode_map(&tmA, grad_out, 2, dims, str, box)) return MM_ERR_CUDA;
  }
  if ((Nw % 64) == 0) {
    uint64_t dims[4] = {64, (uint64_t)rows_cap, (uint64_t)Nw / 64, 1};
    uint64_t str[3] = {(uint64_t)ld_in * 2, 128, (uint64_t)ld_in * 2 * (uint64_t)rows_cap};
    uint32_t box[4] = {64, 64, (uint32_t)(pair == 1 ? 2 : 4), 1};
    if (!encode_map(&tmB, orig_in, 4, dims, str, box)) return MM_ERR_CUDA;
    p.b_multibox = 1;
  } else {
    uint64_t dims[3] = {(uint64_t)Nw, (uint64_t)rows_cap, 1};
    uint64_t str[2] = {(uint64_t)ld_in * 2, (uint64_t)ld_in * 2 * (uint64_t)rows_cap};
    uint32_t box[3] = {64, 64, 1};
    if (!encode_map(&tmB, orig_in, 3, dims, str, box)) return MM_ERR_CUDA;
  }
  p.kind = kGroupedReduce;
  p.epi = kEpiStore;
  p.num_groups = num_groups;
  p.N = Nw;
  p.Mw = Mw;
  p.a_mn = 1;
  p.b_mn = 1;
  if (pair < 0 || pair > 2) {
    set_error("mm_grouped_wgrad: tile mode %d is not one of 0 (single), 1 (pair), 2 (single, unit walk)",
              pair);
    return MM_ERR_ARG;
  }
  p.pair = pair == 1 ? 1 : 0;
  p.unit_walk = pair == 2 ? 1 : 0;
  p.idesc = make_idesc_bf16(p.pair ? 2 * kBlockM : kBlockM, kBlockN, 1, 1);
  p.m_tiles = p.pair ? (Mw + 2 * kBlockM - 1) / (2 * kBlockM) : (Mw + kBlockM - 1) / kBlockM;
  p.n_tiles = (Nw + kBlockN - 1) / kBlockN;
  p.group_offs = group_offs;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.out_group_stride = out_group_stride;
  p.status = reinterpret_cast<StatusRecord*>(status);
  p.tma_store = 1;
  {
    const char* env = getenv("MM_WGRAD_STORE");   // "plain" / "wide": row stores instead of TMA
    if (env && env[0] == 'p') p.tma_store = 0;
    if (env && env[0] == 'w') { p.tma_store = 0; p.wide_store = 1; }
  }
  return launch(tmA, tmB, tmC, p, grid_limit, stream);
}

#ifdef MM_PROFILE
// Instrumented builds only: where the following GEMM launches write their wait counters.
void mm_profile_buffer(void* buffer) { mm::g_prof_buffer = reinterpret_cast<unsigned long long*>(buffer); }
#endif

}  // extern "C"
