/* nvm_parallel_queue.h -- the parallel queue protocol under the reference's header name:
 * get_cid, put_cid, sq_enqueue, sq_dequeue, cq_poll, cq_dequeue (include/nvm_parallel_queue.h there), with
 * the reference's parameter lists; cq_poll returns the command's NVMe status instead of a queue position. */
#ifndef BAM_COMPAT_NVM_PARALLEL_QUEUE_H
#define BAM_COMPAT_NVM_PARALLEL_QUEUE_H
#include "bam/queue.cuh"
using bam::cq_dequeue;
using bam::cq_poll;
using bam::get_cid;
using bam::put_cid;
using bam::sq_dequeue;
using bam::sq_enqueue;
#endif
