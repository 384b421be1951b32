// SeqMSE reconstruction loss (placeholder until the tcgen05 kernel lands in this file).
#include "common.cuh"

extern "C" int64_t aimet_b200_seqmse_scratch_bytes(int64_t, int64_t, int64_t, int32_t) { return 0; }

extern "C" int aimet_b200_seqmse_linear_loss(const void *, const void *, const void *, const void *, int64_t,
                                             int64_t, int64_t, int32_t, int, int, int, float *, int32_t *,
                                             void *, int64_t, void *) {
    return ab::fail(AB_ERR_UNSUPPORTED, "seqmse_linear_loss is not built yet");
}
