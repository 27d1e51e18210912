// MoonEP load-balancing tables: the arithmetic shared by the device kernels and the host entry
// points of moonep.cu.
//
// MoonEP is the reference's remedy for skewed routing.  From the [R, E] matrix of routes per
// (source rank, logical expert), every rank derives the same plan:
//   B.0  routes per expert and per home rank;
//   B.1  "single-source fill": while a rank has a surplus and a rank has a deficit, the rank
//        with the largest surplus fills the whole deficit of the rank with the largest
//        deficit (it may go below its own capacity and be filled later); lowest index wins ties;
//   B.2  a home rank serves its quotas largest first, each time from the local expert with
//        the most routes left (lowest index wins ties); the remainder stays at home;
//   B.3  a rank gives replica slots to its remote experts with routes, most routes first,
//        the LARGER expert id first among equals;
// and from the plan the balanced count cube (how many routes source s sends to physical slot
// p of rank d; physical slots are the E/R home slots followed by E/R replica slots) and, per
// route, its bucket and its position in the bucket-major send order.
// Reference: src/mega_moe/runtime/moonep_planning.py:112-276 (host),
// src/mega_moe/kernels/moonep_planning.py:26-362 (device), and
// src/mega_moe/runtime/balanced_routing.py:274-315, 620-720 (count cube, route placement).
//
// The functions are written once for both sides.  Work that a group of threads shares takes
// a "team": SerialTeam runs it with one thread (host code, or one device thread), WarpTeam
// (device only) spreads the searches over the 32 lanes of a warp; the control flow and the
// updates are the same code.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define MM_HD __host__ __device__ __forceinline__
#else
#define MM_HD inline
#endif

namespace mm {
namespace moonep {

constexpr int kMaxWorld = 64;
constexpr int32_t kInt32Max = 2147483647;

// Why a plan fell back to "every expert stays at home" (status record: code 4, site = reason).
enum PlanReject : int32_t {
  kPlanOk = 0,
  kPlanBadCount = 1,      // a count is negative
  kPlanUnequalRows = 2,   // the source ranks do not all hold the same number of routes
  kPlanNotDropless = 3,   // a rank's histogram total differs from its unfiltered route count
  kPlanTooLarge = 4,      // an expert's global count or a rank's total exceeds int32
  kPlanFillFailed = 5,    // B.1 did not reach zero balances
  kPlanCutFailed = 6,     // B.2 ran out of routes for a quota
  kPlanReplicaBudget = 7  // a rank would need more than E/R replica slots
};

struct MaxAt {
  int32_t value;
  int32_t index;  // -1: no candidate
};

// a beats b: larger value, or equal value and lower (kFirst) / higher (!kFirst) index
template <bool kFirst>
MM_HD bool beats(const MaxAt& a, const MaxAt& b) {
  if (b.index < 0) return a.index >= 0;
  if (a.index < 0) return false;
  if (a.value != b.value) return a.value > b.value;
  return kFirst ? a.index < b.index : a.index > b.index;
}

struct SerialTeam {
  MM_HD bool leader() const { return true; }
  MM_HD int first() const { return 0; }
  MM_HD int step() const { return 1; }
  MM_HD void sync() const {}
  template <bool kFirst>
  MM_HD MaxAt best(MaxAt mine) const {
    return mine;
  }
  MM_HD int32_t sum(int32_t mine) const { return mine; }
};

#if defined(__CUDACC__)
// One warp; every lane must call each member (they synchronise the warp).
struct WarpTeam {
  int lane;
  MM_HD bool leader() const { return lane == 0; }
  MM_HD int first() const { return lane; }
  MM_HD int step() const { return 32; }
  MM_HD void sync() const {
#if defined(__CUDA_ARCH__)
    __syncwarp();
#endif
  }
  template <bool kFirst>
  MM_HD MaxAt best(MaxAt mine) const {
#if defined(__CUDA_ARCH__)
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      MaxAt other;
      other.value = __shfl_xor_sync(0xffffffffu, mine.value, d);
      other.index = __shfl_xor_sync(0xffffffffu, mine.index, d);
      if (beats<kFirst>(other, mine)) mine = other;
    }
#endif
    return mine;
  }
  MM_HD int32_t sum(int32_t mine) const {
#if defined(__CUDA_ARCH__)
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, d);
#endif
    return mine;
  }
};
#endif

// Largest of v[0..n), lowest index among equals; every member of the team gets the result.
template <class Team>
MM_HD MaxAt argmax_first(const Team& team, const int32_t* v, int n) {
  MaxAt mine = {0, -1};
  for (int i = team.first(); i < n; i += team.step()) {
    const MaxAt c = {v[i], i};
    if (beats<true>(c, mine)) mine = c;
  }
  return team.template best<true>(mine);
}

// Largest of v[0..n) outside [skip_lo, skip_hi) that comes after `bound` in the order
// "larger value first, larger index first among equals"; bound.index < 0 = no bound.
template <class Team>
MM_HD MaxAt argmax_last_after(const Team& team, const int32_t* v, int n, int skip_lo, int skip_hi,
                              MaxAt bound) {
  MaxAt mine = {0, -1};
  for (int i = team.first(); i < n; i += team.step()) {
    if (i >= skip_lo && i < skip_hi) continue;
    const MaxAt c = {v[i], i};
    if (bound.index >= 0 && !beats<false>(bound, c)) continue;
    if (beats<false>(c, mine)) mine = c;
  }
  return team.template best<false>(mine);
}

// ---- B.0 -------------------------------------------------------------------------------
// Routes of expert e over all source ranks of counts[world, stride]; `negative` is raised if
// a cell is below zero.
MM_HD int64_t expert_total(const int32_t* counts, int stride, int world, int e, bool* negative) {
  int64_t total = 0;
  for (int s = 0; s < world; ++s) {
    const int32_t c = counts[(int64_t)s * stride + e];
    if (c < 0) *negative = true;
    total += c;
  }
  return total;
}

// ---- B.1 (one thread) --------------------------------------------------------------------
// balance[h] = routes homed on rank h minus the common capacity, consumed; transfers[h * world
// + d] (zeroed by the caller) receives the routes rank h hands to rank d.
MM_HD int32_t fill_deficits(int64_t* balance, int32_t* transfers, int world) {
  for (int round = 0; round <= world; ++round) {
    int giver = 0, taker = 0;
    for (int h = 1; h < world; ++h) {
      if (balance[h] > balance[giver]) giver = h;
      if (balance[h] < balance[taker]) taker = h;
    }
    if (balance[giver] <= 0 || balance[taker] >= 0) break;
    const int64_t amount = -balance[taker];
    if (amount > kInt32Max) return kPlanTooLarge;
    transfers[giver * world + taker] = (int32_t)amount;
    balance[giver] -= amount;
    balance[taker] = 0;
  }
  for (int h = 0; h < world; ++h)
    if (balance[h] != 0) return kPlanFillFailed;
  return kPlanOk;
}

// ---- B.2 (one team per home rank) ----------------------------------------------------------
// allocation[world, num_experts]: on entry the home rank's own row holds the global counts of
// its experts and the other rows' cells of those experts are zero; quota[world] is the home
// rank's row of the transfer matrix and is consumed.
template <class Team>
MM_HD int32_t cut_home_group(const Team& team, int home, int world, int epr, int num_experts,
                             int32_t* quota, int32_t* allocation) {
  int32_t* left = allocation + (int64_t)home * num_experts + (int64_t)home * epr;
  // every round empties a quota or an expert, so world + epr rounds suffice
  for (int round = 0; round <= world + epr; ++round) {
    const MaxAt q = argmax_first(team, quota, world);
    if (q.index < 0 || q.value <= 0) return kPlanOk;
    const MaxAt l = argmax_first(team, left, epr);
    if (l.index < 0 || l.value <= 0) return kPlanCutFailed;
    const int32_t amount = q.value < l.value ? q.value : l.value;
    if (team.leader()) {
      quota[q.index] -= amount;
      left[l.index] -= amount;
      allocation[(int64_t)q.index * num_experts + (int64_t)home * epr + l.index] += amount;
    }
    team.sync();
  }
  return kPlanCutFailed;
}

// ---- B.3 (one team per destination rank) ---------------------------------------------------
// experts_to_copy[dest, 0..epr) and inverse[dest, 0..num_experts) must hold -1 on entry.
// Returns the number of remote experts with routes on `dest`; more than epr of them do not fit
// and the surplus gets no slot (the caller rejects the plan).
template <class Team>
MM_HD int32_t choose_replicas(const Team& team, int dest, int epr, int num_experts,
                              const int32_t* allocation, int32_t* experts_to_copy,
                              int32_t* inverse) {
  const int32_t* row = allocation + (int64_t)dest * num_experts;
  const int home_lo = dest * epr, home_hi = home_lo + epr;
  int32_t mine = 0;
  for (int e = team.first(); e < num_experts; e += team.step())
    if ((e < home_lo || e >= home_hi) && row[e] > 0) ++mine;
  const int32_t needed = team.sum(mine);
  MaxAt prev = {0, -1};
  for (int slot = 0; slot < epr; ++slot) {
    const MaxAt pick = argmax_last_after(team, row, num_experts, home_lo, home_hi, prev);
    if (pick.index < 0 || pick.value <= 0) break;
    if (team.leader()) {
      experts_to_copy[(int64_t)dest * epr + slot] = pick.index;
      inverse[(int64_t)dest * num_experts + pick.index] = slot;
    }
    prev = pick;
  }
  team.sync();
  return needed;
}

// ---- allocation prefix ---------------------------------------------------------------------
// alloc_cumsum[e, d] = routes of expert e executed on ranks 0..d.
MM_HD void allocation_prefix(const int32_t* allocation, int world, int num_experts, int e,
                             int32_t* alloc_cumsum) {
  int32_t run = 0;
  for (int d = 0; d < world; ++d) {
    run += allocation[(int64_t)d * num_experts + e];
    alloc_cumsum[(int64_t)e * world + d] = run;
  }
}

// ---- balanced count cube -----------------------------------------------------------------
// Logical expert behind physical slot `slot` of rank d, -1 for an empty replica slot.
MM_HD int32_t slot_expert(const int32_t* experts_to_copy, int epr, int d, int slot) {
  return slot < epr ? d * epr + slot : experts_to_copy[(int64_t)d * epr + (slot - epr)];
}

// Physical slot of expert e on rank d, -1 if it has none there.
MM_HD int32_t physical_slot(const int32_t* inverse, int num_experts, int epr, int d, int e) {
  if (e / epr == d) return e % epr;
  const int32_t r = inverse[(int64_t)d * num_experts + e];
  return r < 0 ? -1 : epr + r;
}

// The `world` cells of bucket (d, slot): the routes of an expert are numbered source-major;
// source s owns [lo_s, hi_s), rank d executes [alloc_cumsum[e, d-1], alloc_cumsum[e, d]); a
// cell is the length of the overlap.  out[s * out_stride + d * 2 * epr + slot].
MM_HD void bucket_cells(const int32_t* counts, int stride, int world, int num_experts, int epr,
                        const int32_t* alloc_cumsum, const int32_t* experts_to_copy, int d,
                        int slot, int32_t* out, int out_stride) {
  const int bucket = d * 2 * epr + slot;
  const int32_t e = slot_expert(experts_to_copy, epr, d, slot);
  if (e < 0 || e >= num_experts) {
    for (int s = 0; s < world; ++s) out[(int64_t)s * out_stride + bucket] = 0;
    return;
  }
  const int64_t alloc_lo = d ? alloc_cumsum[(int64_t)e * world + d - 1] : 0;
  const int64_t alloc_hi = alloc_cumsum[(int64_t)e * world + d];
  int64_t lo = 0;
  for (int s = 0; s < world; ++s) {
    const int64_t hi = lo + counts[(int64_t)s * stride + e];
    const int64_t a = lo > alloc_lo ? lo : alloc_lo;
    const int64_t b = hi < alloc_hi ? hi : alloc_hi;
    out[(int64_t)s * out_stride + bucket] = b > a ? (int32_t)(b - a) : 0;
    lo = hi;
  }
}

// Routes of expert e held by ranks below `rank`.
MM_HD int32_t lower_rank_routes(const int32_t* counts, int stride, int rank, int e) {
  int32_t total = 0;
  for (int s = 0; s < rank; ++s) total += counts[(int64_t)s * stride + e];
  return total;
}

// ---- route placement -----------------------------------------------------------------------
struct Placement {
  int32_t bucket;    // destination rank * 2 * epr + physical slot, -1: no allocation holds it
  int32_t position;  // row in the bucket-major send order
};

// Route number i of the expert-major stable order, an instance of expert e.
// expert_start[e]: first index of expert e in that order; below[e]: lower_rank_routes.
// Returns the bucket (destination rank * 2 * epr + physical slot, -1 if no allocation or slot
// holds the route); *ordinal_out / *share_lo_out: the route's number among all routes of the
// expert, and the first such number this rank sends to that bucket.
MM_HD int32_t route_bucket(int i, int e, int world, int num_experts, int epr,
                           const int32_t* expert_start, const int32_t* below,
                           const int32_t* alloc_cumsum, const int32_t* inverse,
                           int32_t* ordinal_out, int32_t* share_lo_out) {
  const int32_t ordinal = below[e] + (i - expert_start[e]);
  const int32_t* prefix = alloc_cumsum + (int64_t)e * world;
  int dest = 0;
  while (dest < world && prefix[dest] <= ordinal) ++dest;  // the prefix is non-decreasing
  if (dest >= world) return -1;
  const int32_t slot = physical_slot(inverse, num_experts, epr, dest, e);
  if (slot < 0) return -1;
  const int32_t alloc_lo = dest ? prefix[dest - 1] : 0;
  *ordinal_out = ordinal;
  *share_lo_out = below[e] > alloc_lo ? below[e] : alloc_lo;
  return dest * 2 * epr + slot;
}

MM_HD Placement place_route(int i, int e, int world, int num_experts, int epr,
                            const int32_t* expert_start, const int32_t* below,
                            const int32_t* alloc_cumsum, const int32_t* inverse,
                            const int32_t* send_bucket_starts) {
  Placement p = {-1, -1};
  int32_t ordinal = 0, share_lo = 0;
  p.bucket = route_bucket(i, e, world, num_experts, epr, expert_start, below, alloc_cumsum,
                          inverse, &ordinal, &share_lo);
  if (p.bucket >= 0) p.position = send_bucket_starts[p.bucket] + (ordinal - share_lo);
  return p;
}

}  // namespace moonep
}  // namespace mm
