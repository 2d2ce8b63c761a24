/* nvm_parallel_queue.h -- the parallel queue protocol under the reference's header name:
 * get_cid, put_cid, sq_enqueue, cq_poll, cq_dequeue (include/nvm_parallel_queue.h there). */
#ifndef BAM_COMPAT_NVM_PARALLEL_QUEUE_H
#define BAM_COMPAT_NVM_PARALLEL_QUEUE_H
#include "bam/queue.cuh"
using bam::cq_dequeue;
using bam::cq_poll;
using bam::get_cid;
using bam::put_cid;
using bam::sq_enqueue;
#endif
