/* bafs_ptr.h -- bafs_ptr<T> under the reference's header name (include/bafs_ptr.h:17-132 there). */
#ifndef BAM_COMPAT_BAFS_PTR_H
#define BAM_COMPAT_BAFS_PTR_H
#include "page_cache.h"
#endif
