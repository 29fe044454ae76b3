// Tuned decode-attention kernel (placeholder until the tiled kernel lands).
#include "mz_decode.cuh"

bool mz_decode_tiles_supported(const MzDecodeParams&) { return false; }
int mz_decode_units_tiles(const mz_kv_store& s) { return s.k_groups + (s.res_len + s.group - 1) / s.group; }
int mz_launch_decode_tiles(const MzDecodeParams&, cudaStream_t) { return mz_fail(MZ_ERR_UNSUPPORTED, "tiled kernel not built"); }
