/*
 * C ABI of libmegamoe_sm100.so: the sm_100a kernels behind the `mega_moe` Python
 * operator (expert-parallel MoE layer: routing metadata, dispatch, FC1 + weighted
 * gated activation, FC2 + combine, top-k reduce, and the five backward stages).
 *
 * The reference implementation (Mega-MoE-TD) has no foreign-function boundary of
 * its own: its Python operator launches Triton-Ascend kernels directly.  Each entry
 * point below therefore names the reference *launch site* it stands in for
 * (path:line inside the reference project).  `mega_moe/_native.py` binds all of them
 * with ctypes.
 *
 * Conventions
 *   - every function returns 0 (MM_OK) or a negative MM_ERR_* code and never throws;
 *     mm_last_error() returns the message of the calling thread's last failure;
 *   - all pointers are device pointers unless a parameter says "host";
 *   - the library never takes ownership of caller memory;
 *   - kernels are enqueued on `stream` and the call returns without synchronising,
 *     unless the comment says "synchronous";
 *   - bf16 tensors are passed as void*, int32 index tables as int32_t*;
 *   - device-side waits are bounded: a wait that runs out writes an mm_status_record
 *     into the caller's status buffer and the kernel returns normally.
 */
#ifndef MEGA_MOE_B200_H_
#define MEGA_MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef __CUDA_RUNTIME_H__
typedef struct CUstream_st* cudaStream_t;
#endif

enum {
  MM_OK = 0,
  MM_ERR_ARG = -1,   /* invalid argument (shape, alignment, null pointer) */
  MM_ERR_CUDA = -2,  /* a CUDA runtime / driver call failed */
  MM_ERR_LIMIT = -3  /* request exceeds a fixed limit of the entry point */
};

/* Activation selector shared by forward and backward (reference: config.py:28-32). */
enum { MM_ACT_SWIGLU = 0, MM_ACT_SITUGLU = 1, MM_ACT_CLAMP_SWIGLU = 2 };

/* Format of saved FC1 rows (reference: config.py:179-186 `save_fc1_dtype`,
 * kernels/fused_forward.py:877-949): raw bf16, a plain fp16 copy, or fp8 E4M3 with one fp32
 * scale per row and per `scale_group` columns, table [rows, 2F / scale_group], gate groups
 * first; scale = group amax / 448, an all-zero group keeps q = 0 and the scale 1 / 448. */
enum { MM_FC1_BF16 = 0, MM_FC1_FP16 = 1, MM_FC1_FP8 = 2 };

/* Device status record (32 bytes).  code: 0 ok, 1 wait timed out, 2 receive-capacity
 * overflow, 3 bad index, 4 the load-balancing planner rejected its input and planned "every
 * expert stays at home" (site = MM_PLAN_* reason).  Mirrors the reference's bounded-spin
 * diagnostic record (kernels/dispatch_fc2_bwd.py:23-42). */
typedef struct mm_status_record {
  int32_t code, site, slot, want, seen, block, pad0, pad1;
} mm_status_record;

/* ---- library ---------------------------------------------------------------- */
int mm_abi_version(void);
const char* mm_last_error(void);
/* Number of SMs of the current device (persistent grids are sized from it; stands in
 * for the AICore-count query of config.py:37-62). */
int mm_num_sms(int* out_host);

/* ---- status ------------------------------------------------------------------ */
int mm_status_reset(void* status, cudaStream_t stream);
/* synchronous: waits for `stream`, then copies the record to host memory */
int mm_status_read(const void* status, mm_status_record* out_host, cudaStream_t stream);

/* ---- symmetric buffers over CUDA IPC (reference: runtime/workspace.py:159-222,
 *      aclshmem_create_tensor / aclshmem_free_tensor) ----------------------------- */
int mm_symm_alloc(size_t bytes, void** dptr_host, unsigned char handle_host[64]);
int mm_symm_open(const unsigned char handle_host[64], void** peer_ptr_host);
int mm_symm_close(void* peer_ptr);
int mm_symm_free(void* dptr);

/* Cross-rank barrier through flag words in symmetric memory: writes `epoch` into slot
 * [rank] of every peer's flag array, then waits (bounded) until all `world` slots of the
 * local array hold a value >= epoch.  peer_flags: device array of `world` pointers.
 * phase 0 does both halves; phase 1 only signals and phase 2 only waits, so that work which
 * touches no peer-written memory can run between the two.
 * Stands in for libshmem_device.barrier_all_vec() (runtime/routing.py:91,142). */
int mm_rank_barrier(int32_t* const* peer_flags, int rank, int world, int epoch, int phase,
                    void* status, cudaStream_t stream);

/* ---- routing metadata --------------------------------------------------------- */
/* Scratch bytes mm_route_local needs for `num_routes` routes and `bins` count bins. */
size_t mm_route_scratch_bytes(int num_routes, int bins);

/* Route filter + stable expert-major sort + local count row
 * (reference: runtime/routing.py:635-671 and kernels/fused_forward.py:158-190,307-447).
 *   selected        [num_routes] flat [T, k] expert ids; valid iff 0 <= id < num_experts
 *   send_route      [num_routes] out: flat route id of each send row (valid prefix)
 *   send_token      [num_routes] out: route id / top_k
 *   send_bucket     [num_routes] out: expert id of each send row
 *   route_to_send   [num_routes] out: inverse permutation, -1 for dropped routes
 *   count_row       [bins] out: routes per expert, zero padded
 *   local_stats     [2] out: {number of valid routes, 0}
 */
int mm_route_local(const int32_t* selected, int num_routes, int top_k, int num_experts, int bins,
                   int32_t* send_route, int32_t* send_token, int32_t* send_bucket,
                   int32_t* route_to_send, int32_t* count_row, int32_t* local_stats, void* scratch,
                   size_t scratch_bytes, cudaStream_t stream);

/* Same work and outputs as mm_route_local for callers that cannot allocate device memory
 * (a server with a frozen memory pool, a plugin that owns no allocator): the scratch lives
 * in a 1 MiB array inside the library's device image instead of being passed in.  No
 * counterpart in the reference, whose callers always allocate through the framework.
 * Returns MM_ERR_LIMIT when mm_route_scratch_bytes(num_routes, bins) exceeds 1 MiB.  The first
 * call on a device resolves the array's address; make it before any stream capture.  Calls
 * on one device share the array, so calls that may overlap on the GPU must be ordered.  The
 * call itself allocates nothing. */
int mm_route_local_static(const int32_t* selected, int num_routes, int top_k, int num_experts,
                          int bins, int32_t* send_route, int32_t* send_token,
                          int32_t* send_bucket, int32_t* route_to_send, int32_t* count_row,
                          int32_t* local_stats, cudaStream_t stream);

/* Count exchange (reference: the count publication inside the forward kernel,
 * kernels/fused_forward.py:158-238; on the host path the all_gather of
 * runtime/routing.py:164-192).  Stores this rank's count_row [bins] into row `rank` of every
 * rank's count cube (peer_cubes[d] + cube_offset is rank d's [world, bins] cube), flags it with
 * `epoch` in peer_flags[d][rank] and waits, bounded, until my_flags[0..world) all carry
 * `epoch`; afterwards this rank's cube is complete.  `epoch` must grow with every call; two
 * cubes used alternately (cube_offset) keep a fast rank's next row out of a cube that a slow
 * rank is still reading.  One small kernel, no host synchronisation. */
int mm_count_exchange(const int32_t* count_row, int bins, int rank, int world,
                      int32_t* const* peer_cubes, int64_t cube_offset,
                      int32_t* const* peer_flags, const int32_t* my_flags, int epoch,
                      void* status, cudaStream_t stream);

/* Offsets from the replicated count cube [world, bins]
 * (reference: runtime/routing.py:93-140,318-416; kernels/fused_forward.py:241-304,337-358,
 * 450-480).  Also builds the 128-row tile table of the grouped GEMMs (the counterpart of
 * ops/_torch_forward.py:103-128) and, per received row, the source rank and the row's
 * position in that source's send order (kernels/fc2_combine.py:82-136).
 *   send_bucket_starts, send_bucket_dst_starts   [world * epr]
 *   recv_counts_re [world, epr]   recv_per_expert [epr]   recv_expert_offs [epr + 1]
 *   recv_seg_starts [epr, world + 1]   pull_dst_start [epr * world]
 *   stats [2 + world] = {M, max over destinations, per-destination totals}
 *   mtile_group / mtile_row0 [capacity_rows / 128 + epr]   num_mtiles [1]   (128-row tiles)
 *   mtile2_group / mtile2_row0 [capacity_rows / 256 + epr]  num_mtiles2 [1]  (256-row tiles of
 *     the CTA-pair and skinny GEMMs, mm_gemm_desc.pair = 1 or 2)
 *   row_src_rank / row_src_pos [capacity_rows]
 *   order_prefix [world * epr + 1]: prefix of the local counts in dispatch order (local expert
 *     slot outermost, destination rank rotated by `rank`), bucket_done [world * epr]: zeroed
 *     delivery counters; both feed mm_dispatch_desc
 *   row_arrival / arrival_row [capacity_rows], both or neither (may be null): the permutation
 *     between this receive order (expert-major, then source) and the source-major arrival
 *     order of an all-to-all, and its inverse: the saved contract's local_sort_idxs / inv_local
 *     (ops/_single_saved_adapter.py:335-338)
 * If a destination's total exceeds capacity_rows the status record gets code 2, num_mtiles and
 * num_mtiles2 are 0 and no entry of the row-tile tables is written. */
int mm_route_finalize(const int32_t* count_cube, int rank, int world, int epr, int bins,
                      int capacity_rows, int32_t* send_bucket_starts,
                      int32_t* send_bucket_dst_starts, int32_t* recv_counts_re,
                      int32_t* recv_per_expert, int32_t* recv_expert_offs,
                      int32_t* recv_seg_starts, int32_t* pull_dst_start, int32_t* stats,
                      int32_t* mtile_group, int32_t* mtile_row0, int32_t* num_mtiles,
                      int32_t* mtile2_group, int32_t* mtile2_row0, int32_t* num_mtiles2,
                      int32_t* row_src_rank, int32_t* row_src_pos, int32_t* order_prefix,
                      int32_t* bucket_done, int32_t* row_arrival, int32_t* arrival_row,
                      void* status, cudaStream_t stream);

/* ---- MoonEP load-balancing tables ---------------------------------------------------- */
/* The reference's remedy for skewed routing (runtime/moonep_planning.py, runtime/
 * balanced_routing.py): routes of an overloaded home rank are executed on under-loaded ranks,
 * in replica slots that follow the E/R home slots of a rank (2 * E/R physical slots per rank).
 * These entry points build the integer tables; they sit between mm_count_exchange and
 * mm_route_finalize, which then runs on the balanced cube with epr = 2 * E/R:
 *   mm_route_local -> mm_count_exchange -> mm_moonep_plan -> mm_moonep_count_cube
 *   -> mm_route_finalize(cube, epr = 2 * E/R) -> mm_moonep_map_routes.
 * Each has a *_host twin that runs the same arithmetic on host memory (all pointers host
 * pointers, no stream): the counterpart of the reference's host planner, which takes CPU
 * tensors (runtime/moonep_planning.py:239-276). */
enum {
  MM_PLAN_OK = 0,
  MM_PLAN_BAD_COUNT = 1,      /* a count is negative */
  MM_PLAN_UNEQUAL_ROWS = 2,   /* source ranks hold different numbers of routes */
  MM_PLAN_NOT_DROPLESS = 3,   /* a rank's histogram total differs from its unfiltered count */
  MM_PLAN_TOO_LARGE = 4,      /* an expert's global count or a rank's total exceeds int32 */
  MM_PLAN_FILL_FAILED = 5,    /* B.1 did not reach zero balances */
  MM_PLAN_CUT_FAILED = 6,     /* B.2 ran out of routes for a quota */
  MM_PLAN_REPLICA_BUDGET = 7  /* a rank would need more than E/R replica slots */
};

/* Planning steps B.0-B.3 (reference: runtime/moonep_planning.py:112-276 on the host,
 * kernels/moonep_planning.py:365-460 as four launches; here one launch of one CTA).
 *   counts          [world, stride] routes per (source rank, logical expert); the replicated
 *                   count cube of mm_count_exchange.  total_bin >= 0 names a column that holds
 *                   each rank's unfiltered route count (the dropless check of
 *                   runtime/routing.py:457-481); -1: no such column
 *   allocation      [world, num_experts] out: routes of expert e executed on rank d
 *   alloc_cumsum    [num_experts, world] out: inclusive prefix of `allocation` over ranks
 *   experts_to_copy [world, E/R] out: logical expert in each replica slot, -1 = empty
 *   inverse         [world, num_experts] out: replica slot of expert e on rank d, -1 = none
 *   replica_counts  [world] out: remote experts with routes on each rank
 *   plan_stats      [4] out: {routes per source rank, MM_PLAN_* reason, max of replica_counts, 0}
 * An input the planner cannot balance (reason != 0) yields the plan that keeps every expert
 * at home, and status code 4.  world <= 64, num_experts <= 4096 and divisible by world. */
int mm_moonep_plan(const int32_t* counts, int stride, int world, int num_experts, int total_bin,
                   int32_t* allocation, int32_t* alloc_cumsum, int32_t* experts_to_copy,
                   int32_t* inverse, int32_t* replica_counts, int32_t* plan_stats, void* status,
                   cudaStream_t stream);
int mm_moonep_plan_host(const int32_t* counts, int stride, int world, int num_experts,
                        int total_bin, int32_t* allocation, int32_t* alloc_cumsum,
                        int32_t* experts_to_copy, int32_t* inverse, int32_t* replica_counts,
                        int32_t* plan_stats);

/* Balanced count cube (reference: runtime/balanced_routing.py:274-315,
 * kernels/balanced_routing.py `_kernel_build_balanced_count_cube`): cube[s, d * 2 * E/R + p] =
 * routes source s sends to physical slot p of rank d, every rank computes the whole cube from
 * the replicated counts and the plan.  Columns from world * 2 * E/R to cube_stride are zeroed.
 * Also, for this rank: expert_start [num_experts] = first index of each expert in the
 * expert-major send order of mm_route_local, below [num_experts] = routes of each expert held
 * by lower ranks.  `cube` must not alias `counts`. */
int mm_moonep_count_cube(const int32_t* counts, int stride, int rank, int world, int num_experts,
                         const int32_t* alloc_cumsum, const int32_t* experts_to_copy,
                         int32_t* cube, int cube_stride, int32_t* expert_start, int32_t* below,
                         cudaStream_t stream);
int mm_moonep_count_cube_host(const int32_t* counts, int stride, int rank, int world,
                              int num_experts, const int32_t* alloc_cumsum,
                              const int32_t* experts_to_copy, int32_t* cube, int cube_stride,
                              int32_t* expert_start, int32_t* below);

/* Route placement (reference: runtime/balanced_routing.py:620-720 direct scatter,
 * kernels/balanced_routing.py `_kernel_map_balanced_routes`): turns the expert-major send
 * order of mm_route_local (route_in = its send_route, expert_in = its send_bucket, local_stats
 * = its local_stats) into the bucket-major order over physical slots.  send_bucket_starts
 * [world * 2 * E/R] comes from mm_route_finalize on the balanced cube.  Outputs (must not alias
 * the inputs): send_route / send_token / send_bucket [num_routes], bucket = d * 2 * E/R + p;
 * route_to_send [num_routes] is updated in place for the valid routes.  A route without an
 * allocation or a slot is skipped and reported as status code 3 (the host twin counts them
 * in num_misplaced instead). */
int mm_moonep_map_routes(const int32_t* route_in, const int32_t* expert_in,
                         const int32_t* local_stats, int num_routes, int top_k, int world,
                         int num_experts, const int32_t* expert_start, const int32_t* below,
                         const int32_t* alloc_cumsum, const int32_t* inverse,
                         const int32_t* send_bucket_starts, int32_t* send_route,
                         int32_t* send_token, int32_t* send_bucket, int32_t* route_to_send,
                         void* status, cudaStream_t stream);
int mm_moonep_map_routes_host(const int32_t* route_in, const int32_t* expert_in, int num_valid,
                              int num_routes, int top_k, int world, int num_experts,
                              const int32_t* expert_start, const int32_t* below,
                              const int32_t* alloc_cumsum, const int32_t* inverse,
                              const int32_t* send_bucket_starts, int32_t* send_route,
                              int32_t* send_token, int32_t* send_bucket, int32_t* route_to_send,
                              int32_t* num_misplaced);

/* MoonEP as a re-labelling of routes: physical [num_routes] out, physical[route] = d * 2 * E/R + p,
 * the bucket that executes the route, -1 for routes mm_route_local dropped (route_to_send < 0).  Inputs as for
 * mm_moonep_map_routes (expert_start and below from mm_moonep_count_cube).  Running the ordinary
 * routing (mm_route_local, mm_count_exchange, mm_route_finalize) with `physical` as the expert ids
 * of a layer of 2 * E experts yields the balanced send order, count cube and offsets, so the
 * rest of the layer runs unchanged over 2 * E/R groups per rank
 * (reference: the physical-slot forward, ops/_moonep_torch_forward.py:226-430). */
int mm_moonep_relabel_routes(const int32_t* route_in, const int32_t* expert_in,
                             const int32_t* route_to_send, const int32_t* local_stats,
                             int num_routes, int world, int num_experts,
                             const int32_t* expert_start, const int32_t* below,
                             const int32_t* alloc_cumsum, const int32_t* inverse,
                             int32_t* physical, void* status, cudaStream_t stream);

/* One weight (or weight-gradient) table of the replica transport.  `local` is this rank's
 * [E/R][bytes] table of its home experts (experts `local_stride` bytes apart); peer[d] is rank
 * d's replica table [E/R slots][bytes], slots contiguous, in memory every rank can address
 * (mm_symm_alloc / mm_symm_open).  bytes and local_stride are multiples of 16, pointers 16-byte
 * aligned. */
typedef struct mm_replica_table {
  const void* local;
  int64_t local_stride;
  int64_t bytes;
  void* const* peer; /* device array of `world` pointers */
} mm_replica_table;

/* Owner-push of replica weights (reference: kernels/replica_weight_prefetch.py:17-180,
 * runtime/replica_weight_prefetch.py): for every (rank d, slot b) with experts_to_copy[d, b]
 * owned by `rank`, stores that expert's block of weights0 (and weights1, may be null) into slot
 * b of rank d's replica table.  Plain peer stores from a persistent grid (grid_limit 0: two
 * CTAs per SM); no waits.  The destinations may read their slots after a rank barrier that
 * follows this launch on every rank (mm_rank_barrier). */
int mm_moonep_push_replicas(const int32_t* experts_to_copy, int rank, int world, int epr,
                            const mm_replica_table* weights0, const mm_replica_table* weights1,
                            int grid_limit, cudaStream_t stream);

/* Owner-pull of replica weight gradients (reference: kernels/replica_grad_reduce.py:62-190):
 * for every home expert of `rank` with copies elsewhere (inverse[d, e] >= 0, d != rank),
 * grads.local[e] = bf16(fp32(grads.local[e]) + sum over d ascending of fp32(peer[d][slot])),
 * bf16 elements, one rounding.  The tables of the peers are only read.  All ranks must have
 * finished writing their replica gradients (a rank barrier before this launch), and must not
 * overwrite them before every owner has pulled (a rank barrier after it). */
int mm_moonep_pull_replica_grads(const int32_t* inverse, int rank, int world, int epr,
                                 const mm_replica_table* grads0, const mm_replica_table* grads1,
                                 int grid_limit, cudaStream_t stream);

/* ---- dispatch / combine data movement ---------------------------------------------- */
/* Push send row i (= src[send_token[i]]) to rank send_bucket[i] / epr at row
 * send_bucket_dst_starts[b] + (i - send_bucket_starts[b]) of that rank's receive buffer,
 * with its fp32 routing weight alongside when `weights` is not null
 * (reference: kernels/dispatch_fc1.py:365-508; kernels/dispatch_fc2_bwd.py:254-306).
 *   peer_rows / peer_weights: device arrays of `world` base pointers. */
int mm_dispatch_rows(const void* src, int hidden, const float* weights, const int32_t* send_token,
                     const int32_t* send_route, const int32_t* send_bucket,
                     const int32_t* send_bucket_starts, const int32_t* send_bucket_dst_starts,
                     const int32_t* local_stats, int max_routes, int epr, int capacity_rows,
                     void* const* peer_rows, float* const* peer_weights, cudaStream_t stream);

/* out[t] = bf16(sum_j fp32(rows[route_to_send[t*k + j]])) in slot order, -1 skipped
 * (reference: kernels/fused_forward.py:1319-1387).  When gate_in is not null also
 * gate_out[t, j] = gate_in[route_to_send[t*k + j]] (0 for dropped), the routing-weight
 * gradient gather of kernels/combine_fc1_bwd.py:357-394; gate_out_f32 (may be null) receives
 * the same values as fp32, the dtype the router's autograd expects (ops/function.py:207-215). */
int mm_topk_reduce(const void* rows, int64_t ld_rows, const int32_t* route_to_send, int tokens,
                   int top_k, int hidden, void* out, const void* gate_in, void* gate_out,
                   float* gate_out_f32, cudaStream_t stream);

/* ---- grouped GEMMs (tcgen05 / TMEM) ------------------------------------------------- */
typedef struct mm_gemm_desc {
  const void* a;              /* [a_rows_cap, K] bf16 rows grouped by expert */
  int64_t lda;                /* elements between A rows */
  int64_t a_rows_cap;         /* rows the buffer holds (tensor-map extent) */
  const void* b;              /* per-group weights */
  int32_t b_k_major;          /* 1: [g][n][k] with k contiguous; 0: [g][k][n] with n contiguous */
  int32_t b_cols_total;       /* n extent of the weight table (2F for the packed gate|up table) */
  int64_t b_ld;               /* elements between consecutive rows of one group's matrix */
  int64_t b_group_stride;     /* elements between groups */
  int32_t num_groups;
  int32_t N;                  /* output columns (fused FC1: F) */
  int32_t K;                  /* reduction extent */
  int32_t grid_limit;         /* 0: one CTA per SM */
  int32_t pair;               /* tile mode.  0: one CTA per 128-row x 256-column tile (pass the
                                 128-row tile table).  1: tcgen05 cta_group::2 - clusters of two
                                 CTAs share 256-row tiles.  2: "skinny", for groups with few rows:
                                 the product is computed transposed, 256 output columns x up to
                                 256 rows per tile with the rows as the MMA's N extent in steps
                                 of 16.  Modes 1 and 2 take the 256-row tile table. */
  int32_t reserved;
  const int32_t* group_offs;  /* [num_groups + 1] */
  const int32_t* mtile_group; /* from mm_route_finalize */
  const int32_t* mtile_row0;
  const int32_t* num_mtiles;
  void* status;
} mm_gemm_desc;

/* Optional fused dispatch of mm_fc1_swiglu / mm_grouped_gemm: two extra warps of every CTA push
 * this rank's send rows (row i = src[send_token[i]]) into the owning ranks' receive buffers
 * in dispatch order, flag each (source, expert) bucket as complete in the destination's
 * `flags` array (st.release.sys of `epoch`), and the GEMM waits per expert until all `world`
 * sources have flagged it instead of waiting for a rank barrier
 * (reference: dispatch overlapped with FC1, kernels/dispatch_fc1.py:365-508 and
 * kernels/fused_forward.py:483-534,1106-1158).  `epoch` must grow with every fused launch. */
typedef struct mm_dispatch_desc {
  const void* src;                    /* [tokens, hidden] bf16 rows to send */
  const float* weights;               /* [tokens * top_k] fp32, sent alongside; may be null */
  const int32_t* send_token;
  const int32_t* send_route;
  const int32_t* send_bucket_starts;
  const int32_t* send_bucket_dst_starts;
  const int32_t* count_row;           /* rows per bucket (local count row) */
  const int32_t* order_prefix;        /* from mm_route_finalize */
  const int32_t* local_stats;         /* [0] = number of send rows */
  int32_t* bucket_done;               /* [world * epr], zero at launch; left zero again */
  void* const* peer_rows;             /* device array of `world` receive-buffer bases */
  float* const* peer_weights;         /* device array of `world` weight-buffer bases */
  int32_t* const* peer_flags;         /* device array of `world` flag-array bases */
  const int32_t* my_flags;            /* this rank's flag array [world * epr] */
  int32_t hidden, rank, world, epr, capacity_rows, epoch;
} mm_dispatch_desc;

/* FC1 with the weighted gated activation fused in the epilogue
 * (reference: kernels/fused_forward.py:551-876).  b is the packed [E, H, 2F] table
 * (b_k_major = 0, b_cols_total = 2F, N = F).
 *   act_out [rows, F] = bf16(f(bf16(gate), bf16(up)) * row_weight)
 *   raw_out [rows, 2F] = bf16 gate | up (may be null; in tile mode 2 a non-null raw_out
 *     selects the two-step form: a plain GEMM stores the raw rows, a row-wise pass applies
 *     the activation - same rounding points, two launches)
 *   row_weight_bf16_out [rows] = bf16(row_weight), the received routing weights as the
 *     backward reads them (ops/_torch_forward.py:254); may be null
 *   dispatch: null for rows already resident in `a`, else the fused dispatch above */
int mm_fc1_swiglu(const mm_gemm_desc* d, const mm_dispatch_desc* dispatch, void* act_out,
                  int64_t ld_act, void* raw_out, int64_t ld_raw, const float* row_weight,
                  void* row_weight_bf16_out, int activation, float beta, float linear_beta,
                  float clamp_limit, cudaStream_t stream);

/* out[rows of g, 0:N] = bf16(A[rows of g] * B_g)
 * (reference: kernels/dispatch_fc1.py:580-751 for FC1 without activation,
 *  kernels/dispatch_fc2_bwd.py:309-485 for the FC2 input gradient). */
int mm_grouped_gemm(const mm_gemm_desc* d, const mm_dispatch_desc* dispatch, void* out,
                    int64_t ld_out, cudaStream_t stream);

/* Same product, but each output row is stored into rank row_dst_rank[row]'s buffer at row
 * row_dst_pos[row] (reference: FC2 + return, kernels/fused_forward.py:1010-1025,1161-1279;
 * FC1 input gradient + push, kernels/combine_fc1_bwd.py:114-286). */
int mm_grouped_gemm_scatter(const mm_gemm_desc* d, const int32_t* row_dst_rank,
                            const int32_t* row_dst_pos, void* const* peer_bases, int64_t ld_dst,
                            cudaStream_t stream);

/* Weight gradient: out[g][m', n'] = bf16(sum over rows of g: grad_out[row, m'] * orig_in[row, n'])
 * (reference: kernels/transposed_grouped_gemm.py:24-66; kernels/mega_bwd.py:394-493).
 * Groups without rows produce zeros.  `pair`: 0 one CTA per 128x256 tile, every step-th tile;
 * 1 CTA pairs (cta_group::2); 2 one CTA per tile walking whole (group, n-tile) units so that one
 * operand stays in shared memory - for groups of up to 256 rows. */
int mm_grouped_wgrad(const void* grad_out, int64_t ld_go, int32_t Mw, const void* orig_in,
                     int64_t ld_in, int32_t Nw, int64_t rows_cap, const int32_t* group_offs,
                     int32_t num_groups, void* out, int64_t ld_out, int64_t out_group_stride,
                     void* status, int32_t grid_limit, int32_t pair, cudaStream_t stream);

/* ---- backward stage 2 ------------------------------------------------------------- */
/* Gated-activation backward per received row (reference: kernels/swiglu_bwd.py:15-83):
 *   grad_fc1 [rows, 2F] = dGate | dUp (bf16), grad_scale [rows] = bf16(sum f(g) v(u) dC).
 * `num_rows` is read from device memory (stats[0]).  When peer_gate is not null the row's
 * grad_scale is also stored to rank row_dst_rank[row] at peer_gate[rank][row_dst_pos[row]].
 * fc1_out is in `fc1_format` (ld_fc1 in elements); fp8 rows are dequantised at the load with
 * fc1_scale (reference: kernels/mega_bwd.py:3187-3205). */
int mm_swiglu_bwd(const void* grad_act, int64_t ld_ga, const void* fc1_out, int64_t ld_fc1,
                  const void* row_scale_bf16, int ffn, const int32_t* num_rows, int max_rows,
                  void* grad_fc1, int64_t ld_gf, void* grad_scale, int activation, float beta,
                  float linear_beta, float clamp_limit, const int32_t* row_dst_rank,
                  const int32_t* row_dst_pos, void* const* peer_gate, int fc1_format,
                  const float* fc1_scale, int fc1_scale_group, cudaStream_t stream);

/* ---- router in front of the layer ---------------------------------------------------- */
/* selected [tokens, top_k] int32 = the top_k experts of every logits row in descending order
 * of their logits (ties: lower expert id first); weights [tokens, top_k] fp32 = softmax over
 * the selected logits (reference: the post-router inputs of its own benchmark and tests,
 * benchmark/layer/bench_moe_suite.py:487-497).  top_k <= 32, num_experts <= 1024
 * (MM_ERR_LIMIT above). */
int mm_router_topk(const float* logits, int64_t ld_logits, int tokens, int num_experts, int top_k,
                   int32_t* selected, float* weights, cudaStream_t stream);

/* ---- saved-activation formats and the recompute backward ---------------------------- */
/* Convert the raw bf16 FC1 rows [rows, cols = 2F] to the saved format: MM_FC1_FP16 or
 * MM_FC1_FP8 (+ scale table [rows, cols / scale_group])
 * (reference: kernels/fused_forward.py:877-949, quantise leg of the FC1 epilogue). */
int mm_fc1_save_convert(const void* raw_bf16, int64_t ld_raw, int cols, const int32_t* num_rows,
                        int max_rows, int fc1_format, int scale_group, void* out, int64_t ld_out,
                        float* scale, cudaStream_t stream);

/* Recompute the weighted activation rows act [rows, F] = bf16(f(gate, up) * bf16 row scale)
 * from saved FC1 rows of any format (reference: kernels/mega_bwd.py:1408-1465,
 * MOE_SAVED_RECOMPUTE=1). */
int mm_swiglu_recompute(const void* fc1_out, int64_t ld_fc1, int fc1_format, const float* fc1_scale,
                        int fc1_scale_group, const void* row_scale_bf16, int ffn,
                        const int32_t* num_rows, int max_rows, void* act_out, int64_t ld_act,
                        int activation, float beta, float linear_beta, float clamp_limit,
                        cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MEGA_MOE_B200_H_ */
