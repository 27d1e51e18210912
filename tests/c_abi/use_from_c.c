/* A C99 caller of libmegamoe_sm100.so: includes the public header as plain C, takes the address
 * of every entry point (the generated ALL_ENTRY_POINTS list) and runs one that needs no GPU. */
#include <stdio.h>

#include "mega_moe_b200.h"

static const void* const entry_points[] = {ALL_ENTRY_POINTS};

int main(void) {
  /* two ranks, four experts, every route to expert 0: half of them must move to rank 1 */
  int32_t counts[2][4] = {{4, 0, 0, 0}, {4, 0, 0, 0}};
  int32_t allocation[8], alloc_cumsum[8], experts_to_copy[4], inverse[8], replicas[2], stats[4];
  mm_status_record record = {0, 0, 0, 0, 0, 0, 0, 0};
  mm_replica_table table = {0, 0, 0, 0};
  size_t listed = sizeof(entry_points) / sizeof(entry_points[0]);
  int rc = mm_moonep_plan_host(&counts[0][0], 4, 2, 4, -1, allocation, alloc_cumsum,
                               experts_to_copy, inverse, replicas, stats);
  printf("abi=%d entry_points=%lu rc=%d prefix=%d,%d copy=%d reason=%d record=%d table=%d\n",
         mm_abi_version(), (unsigned long)listed, rc, alloc_cumsum[0], alloc_cumsum[1],
         experts_to_copy[2], stats[1], record.code, (int)table.bytes);
  return rc == MM_OK ? 0 : 1;
}
