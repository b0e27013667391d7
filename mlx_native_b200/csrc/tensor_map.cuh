// cuTensorMapEncodeTiled fetched through the runtime (no link against the driver library).
#pragma once
#include <cuda.h>  // CUtensorMap (types only)

namespace mlxn {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
// Null when the driver does not export the encoder.  Defined in qmv_tc.cu.
EncodeTiledFn encode_tiled_fn();

}  // namespace mlxn
