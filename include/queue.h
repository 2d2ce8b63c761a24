/* queue.h -- QueuePair under the reference's header name (include/queue.h:27-53 there).  Queue
 * pairs are created with their controller (bam_ctrl_create), not one by one. */
#ifndef BAM_COMPAT_QUEUE_H
#define BAM_COMPAT_QUEUE_H
#include "bam/abi_types.h"
#define MAX_SQ_ENTRIES_64K 1024          /* deepest queue a controller offers (include/queue.h:55 there) */
#define MAX_CQ_ENTRIES_64K 1024
#endif
