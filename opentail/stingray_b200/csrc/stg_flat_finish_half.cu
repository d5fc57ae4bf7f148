// The small-CTA finish of the flat step's chunked rows, 512 threads, two CTAs per SM.
#define STG_KTHREADS 512
#define STG_SMALL_CTAS 2
#define STG_SMALL_KERNEL k_flat_finish_half
#define STG_SMALL_LAUNCH launch_flat_finish_half
#include "stg_flat_finish_small.inc"
