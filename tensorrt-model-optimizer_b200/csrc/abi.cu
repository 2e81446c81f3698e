// Library-level entry points: status strings, version, device query.
#include "common.cuh"

extern "C" const char* b200q_strerror(int status) {
  switch (status) {
    case B200Q_OK: return "ok";
    case B200Q_ERR_NULL: return "a required pointer is NULL";
    case B200Q_ERR_DTYPE: return "unknown element type code";
    case B200Q_ERR_ALIGN: return "pointer is not aligned as the kernel requires";
    case B200Q_ERR_SHAPE: return "size is not positive or not divisible by the block size";
    case B200Q_ERR_ARG: return "argument out of range";
    case B200Q_ERR_CUDA: return "CUDA runtime error at launch";
    case B200Q_ERR_UNSUPPORTED: return "request not covered by the kernels";
    case B200Q_ERR_TIMEOUT: return "bounded device-side wait ran out";
    case B200Q_ERR_CAPACITY: return "request exceeds the scratch capacity built into the library";
    default: return "unknown status";
  }
}

extern "C" int b200q_version(void) { return 100; }

extern "C" int b200q_sm_count(void) { return b200q::sm_count_cached(); }
