// Version and error-string entry points of libffmoe.
#include "ffm_common.cuh"

extern "C" int ffm_version(void) { return FFM_VERSION; }

extern "C" const char* ffm_error_string(int code) {
  switch (code) {
    case FFM_OK: return "ok";
    case FFM_ERR_BAD_ARG: return "bad argument (null pointer, negative size or unknown enum)";
    case FFM_ERR_UNSUPPORTED: return "shape not supported by the sm_100a kernels (see include/ffmoe.h limits)";
    case FFM_ERR_LAUNCH: return "CUDA launch or driver call failed";
    case FFM_ERR_WORKSPACE: return "workspace too small";
    case FFM_ERR_NO_DRIVER: return "cuTensorMapEncodeTiled not available from the CUDA driver";
    case FFM_ERR_STATIC_LIMIT:
      return "problem exceeds the built-in scratch of ffm_group_rows_static (E <= 256 experts, T <= 1048576 rows)";
    case FFM_STATUS_WAIT_PRODUCER: return "device: TMA producer wait ran out";
    case FFM_STATUS_WAIT_MMA: return "device: MMA issuer wait ran out";
    case FFM_STATUS_WAIT_EPILOGUE: return "device: epilogue wait ran out";
    case FFM_STATUS_BAD_INDEX: return "device: expert index or row position out of range";
    case FFM_STATUS_WAIT_PEER: return "device: a peer GPU did not signal within the wait budget";
    case FFM_STATUS_EP_OVERFLOW: return "device: a rank would receive more rows than the declared bound; nothing was moved";
    default: return "unknown code";
  }
}
