// Chunk-parallel Gated-DeltaNet prefill scan (placeholder translation unit; filled in below).
#include "tt_common.h"

TT_API int tt_gdn_scan_chunked(tt_context *ctx, tt_stream stream, const void *conv_out, const void *a,
                               const void *b, const void *a_log, const void *dt_bias, float *state, void *y,
                               const tt_gdn_shape *shape, uint32_t rows, uint32_t row_stride, uint32_t chunk) {
    TT_ENTER(ctx);
    (void)stream; (void)conv_out; (void)a; (void)b; (void)a_log; (void)dt_bias; (void)state; (void)y;
    (void)shape; (void)rows; (void)row_stride; (void)chunk;
    return tt_set_error(ctx, TT_ERR_UNSUPPORTED_SHAPE, "chunked scan is not built yet");
}
