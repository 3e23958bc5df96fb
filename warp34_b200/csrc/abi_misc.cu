// Library identification for the C ABI.
#include "../../include/warp34_b200.h"

extern "C" const char* warp34_b200_version(void) { return "warp34_b200 0.1 sm_100a"; }
