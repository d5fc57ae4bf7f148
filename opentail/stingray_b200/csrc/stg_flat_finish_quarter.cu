// The small-CTA finish of the flat step's chunked rows, 256 threads, four CTAs per SM.
#define STG_KTHREADS 256
#define STG_SMALL_CTAS 4
#define STG_SMALL_KERNEL k_flat_finish_quarter
#define STG_SMALL_LAUNCH launch_flat_finish_quarter
#include "stg_flat_finish_small.inc"
