// ABI bookkeeping: version and the per-thread error string.
#include "common.cuh"

extern "C" int e3b_abi_version(void) { return 1; }

extern "C" const char* e3b_last_error(void) { return e3b::error_buffer(); }
