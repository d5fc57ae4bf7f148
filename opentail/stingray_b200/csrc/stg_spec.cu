// Speculative verification and vocabulary-sharded entry points (being filled in).
#include "stg_handle.h"

using namespace stg;

extern "C" {

int stg_spec_verify(StgHandle h, const StgSpecBatch *, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_mtp_accept(StgHandle h, const void *, int32_t, int32_t, int32_t, int64_t, const int32_t *, float, int32_t *,
                   int32_t *, float *, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_comm_unique_id(void *) { return STG_ERR_UNSUPPORTED; }
int stg_comm_init(StgHandle h, const void *, int32_t, int32_t) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_comm_destroy(StgHandle) { return STG_OK; }
int stg_shard_select(StgHandle h, const StgSampleBatch *, int32_t, int32_t, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_shard_allgather(StgHandle h, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_shard_finish(StgHandle h, const StgSampleBatch *, int32_t, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }
int stg_shard_gather_local(StgHandle h, const StgHandle *, int32_t, void *) { return fail(h, STG_ERR_UNSUPPORTED, "not built yet"); }

}
